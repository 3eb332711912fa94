// Fused small-MLP inference/forward kernel on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One persistent CTA per SM runs kSlots independent 128-thread "slots"; each slot walks tiles of 128
// input rows.  Per tile and layer one elected thread issues K/16 tcgen05.mma instructions
// (A = activations in shared memory, B = the layer's weights in shared memory, D = fp32 accumulator in
// tensor memory), commits them to an mbarrier, and the slot's four warps then pull their 32 TMEM lanes
// with tcgen05.ld, apply bias + activation in registers and write the bf16 result back into the SAME
// shared-memory buffer as the next layer's A operand (the MMA that read it has completed).  While
// one slot runs its epilogue the tensor core works on another slot's tile.  All weights of the network
// arrive once per CTA with a single TMA bulk copy; input tiles arrive by tiled TMA loads.
//
// This replaces the per-layer cuBLAS GEMMs + elementwise kernels of the reference's nn.Sequential MLPs
// (landmark/nerf_components/model_components/fields/mlp_decoder.py:70-109) and the tiny-cuda-nn
// networks of its fused decoder (fused_mlp_decoder.py:69-90).  The optional "GridNeRF colour" stage
// reproduces benchmarks/nerf/gridnerf/gridnerf.py:137-174: layer 0 is the bias-free basis projection
// (features -> 27), whose output f together with the view direction d is expanded in registers to
// [f, d, sin(f 2^k), cos(f 2^k), sin(d 2^k), cos(d 2^k)] (k = 0, 1) = 150 inputs of the 3-layer decoder.
#include "fused_mlp.cuh"
#include <cstdlib>

namespace lmb {

constexpr int kSlots = 3;
constexpr int kSlotThreads = 128;

// status words: 0 ok, 1 weight load timed out, 2 input tile load timed out, 3 MMA completion timed out
__global__ void __launch_bounds__(kSlots * kSlotThreads, 1)
fused_mlp_kernel(const __grid_constant__ MLPInputs inputs, const unsigned char* __restrict__ blob, MLPSpec spec,
                 const int* __restrict__ count_ptr, long long max_rows, float* __restrict__ out, int out_stride,
                 int* __restrict__ status) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // round the dynamic window up to 1 KB so TMA destinations and operand chunks are well aligned
  unsigned char* smem = smem_raw + ((1024u - (tc05::smem_u32(smem_raw) & 1023u)) & 1023u);
  unsigned char* wsm = smem;                                        // weights + biases
  unsigned char* act_base = smem + ((spec.blob_bytes + 1023) & ~1023);
  __shared__ __align__(8) uint64_t bar_w, bar_in[kSlots], bar_mma[kSlots];
  __shared__ uint32_t tmem_base_sh;
  // per-layer tables: indexed with the run-time layer number, so a copy in shared memory (a kernel parameter indexed
  // dynamically is spilled to local memory, and with the L1 carved down to shared memory every such read goes to L2)
  __shared__ int sK[kMaxLayers], sN[kMaxLayers], sAct[kMaxLayers], sWoff[kMaxLayers], sBoff[kMaxLayers];
  if (threadIdx.x < kMaxLayers) {
    sK[threadIdx.x] = spec.K[threadIdx.x]; sN[threadIdx.x] = spec.N[threadIdx.x]; sAct[threadIdx.x] = spec.act[threadIdx.x];
    sWoff[threadIdx.x] = spec.w_off[threadIdx.x]; sBoff[threadIdx.x] = spec.b_off[threadIdx.x];
  }

  const int tid = threadIdx.x;
  const int slot = tid / kSlotThreads;
  const int row = tid % kSlotThreads;          // row of the tile == TMEM lane owned by this thread
  const int warp_in_slot = row >> 5;
  unsigned char* act = act_base + (size_t)slot * kActBytes;

  if (tid == 0) {
    tc05::mbar_init(&bar_w, 1);
    for (int s = 0; s < kSlots; ++s) { tc05::mbar_init(&bar_in[s], 1); tc05::mbar_init(&bar_mma[s], 1); }
    tc05::fence_barrier_init();
  }
  if (tid < 32) tc05::tmem_alloc(&tmem_base_sh, 512);
  tc05::fence_before_sync();
  __syncthreads();
  tc05::fence_after_sync();
  const uint32_t tmem_slot = tmem_base_sh + (uint32_t)(slot * kSlotCols);
  const uint32_t tmem_lane = tmem_slot + ((uint32_t)(warp_in_slot * 32) << 16);

  if (tid == 0) {
    tc05::mbar_expect_tx(&bar_w, (uint32_t)spec.blob_bytes);
    tc05::tma_bulk_g2s(wsm, blob, (uint32_t)spec.blob_bytes, &bar_w);
  }
  bool ok = tc05::mbar_wait(&bar_w, 0);
  ok = __syncthreads_and(ok);
  if (!ok && tid == 0) atomicExch(status, 1);

  const long long n_rows = resolve_count(count_ptr, max_rows);
  const long long n_tiles = (n_rows + kTileRows - 1) / kTileRows;
  const int in_chunks = spec.in_width >> 3;
  const bool whole_rows = inputs.n128 + inputs.n64 > 0;
  const uint32_t in_bytes = whole_rows ? (uint32_t)(inputs.n128 * kTileRows * 128 + inputs.n64 * kTileRows * 64)
                                       : (uint32_t)(in_chunks * kTileRows * 16);
  const int bar_id = 1 + slot;
  uint32_t ph_in = 0, ph_mma = 0;

  // Input tile of a slot: whole rows in the swizzled layouts (single local source) or one box [8 columns x 128 rows] per
  // 16-byte column chunk (several sources).  Issued by the slot's first thread.
  auto issue_input = [&](long long t) {
    const long long r0 = t * kTileRows;
    tc05::mbar_expect_tx(&bar_in[slot], in_bytes);
    if (whole_rows) {
      for (int a = 0; a < inputs.n128; ++a)
        tc05::tma_load_2d(act + (size_t)a * kTileRows * 128, &inputs.map[0], a * 64, (int)r0, &bar_in[slot]);
      if (inputs.n64)
        tc05::tma_load_2d(act + (size_t)inputs.n128 * kTileRows * 128, &inputs.map[1], inputs.n128 * 64, (int)r0, &bar_in[slot]);
    } else {
      int src = 0;
      for (int c = 0; c < in_chunks; ++c) {
        while (src + 1 < inputs.n_src && c >= inputs.chunk_begin[src + 1]) ++src;
        tc05::tma_load_3d(act + (size_t)c * kTileRows * 16, &inputs.map[src], 0, c - inputs.chunk_begin[src], (int)r0,
                          &bar_in[slot]);
      }
    }
  };
  const long long tile_stride = (long long)gridDim.x * kSlots;
  const long long first_tile = (long long)blockIdx.x * kSlots + slot;
  // The copy of a slot's NEXT tile is issued as soon as the last layer's MMA of the current tile has read the buffer, so
  // it runs under the last epilogue instead of in front of the next tile (measured: 2 500 cycles of exposed wait per tile).
  bool in_flight = ok && first_tile < n_tiles;
  if (in_flight && row == 0) issue_input(first_tile);

  for (long long tile = first_tile; ok && tile < n_tiles; tile += tile_stride) {
    const long long row0 = tile * kTileRows;
    float dir[3] = {0.f, 0.f, 0.f};
    if (spec.pe_stage && whole_rows && row0 + row < n_rows) {
      // the tile arrives in the swizzled layout: the three direction values come from the row in global memory, and
      // the loads are in flight while the thread waits for the tile
      const __nv_bfloat16* dp = inputs.x0 + (row0 + row) * (long long)spec.in_width + spec.dir_col;
#pragma unroll
      for (int i = 0; i < 3; ++i) dir[i] = __bfloat162float(dp[i]);
    }
    bool got = tc05::mbar_wait(&bar_in[slot], ph_in);
    ph_in ^= 1;
    in_flight = false;
    if (!tc05::bar_and(bar_id, kSlotThreads, got)) { if (row == 0) atomicExch(status, 2); ok = false; break; }
    if (spec.pe_stage && !whole_rows) {
#pragma unroll
      for (int i = 0; i < 3; ++i) dir[i] = load_elem(act, spec.dir_col + i, row);
    }

    for (int l = 0; l < spec.n_layers; ++l) {
      const int K = sK[l], N = sN[l];
      // ---- MMA: D[128 x N] = A[128 x K] * W_l^T ----------------------------------------------------
      if (row == 0) {
        tc05::fence_after_sync();
        const uint32_t a_addr = tc05::smem_u32(act);
        const uint32_t b_addr = tc05::smem_u32(wsm + sWoff[l]);
        const uint32_t idesc = tc05::idesc_bf16(N, false, false);
        // One thread issues K/16 MMAs; their shared-memory descriptors differ only in the start-address field (bits
        // 0-13, in 16-byte units), so each step is an add instead of a rebuilt descriptor - this thread's issue loop
        // is in front of every layer of the slot.
        uint64_t db = tc05::smem_desc(b_addr, (uint32_t)(N * 16), 128);
        const uint64_t db_step = (uint64_t)((2 * N * 16) >> 4);             // two 8-column weight chunks per step
        if (l == 0 && whole_rows) {
          int k = 0;
          for (int a = 0; a < inputs.n128 && k < K; ++a) {                   // 64-column pieces, 128-byte swizzle
            uint64_t da = tc05::smem_desc_swizzled(a_addr + (uint32_t)a * (kTileRows * 128), 1024, 2);
            for (int j = 0; j < 4 && k < K; ++j, k += 16) {
              tc05::mma_ss(tmem_slot, da, db, idesc, k > 0);
              da += 2; db += db_step;                                        // 16 columns = 32 bytes inside the row
            }
          }
          if (k < K) {                                                       // last piece, 64-byte swizzle
            uint64_t da = tc05::smem_desc_swizzled(a_addr + (uint32_t)inputs.n128 * (kTileRows * 128), 512, 4);
            for (; k < K; k += 16) {
              tc05::mma_ss(tmem_slot, da, db, idesc, k > 0);
              da += 2; db += db_step;
            }
          }
        } else {
          uint64_t da = tc05::smem_desc(a_addr, kTileRows * 16, 128);
          const uint64_t da_step = (uint64_t)((2 * kTileRows * 16) >> 4);   // two 8-column activation chunks per step
          for (int k = 0; k < K; k += 16) {
            tc05::mma_ss(tmem_slot, da, db, idesc, k > 0);
            da += da_step; db += db_step;
          }
        }
        tc05::mma_commit(&bar_mma[slot]);
      }
      bool done = tc05::mbar_wait(&bar_mma[slot], ph_mma);
      ph_mma ^= 1;
      if (!tc05::bar_and(bar_id, kSlotThreads, done)) { if (row == 0) atomicExch(status, 3); ok = false; break; }
      tc05::fence_after_sync();
      const bool last = (l == spec.n_layers - 1);
      if (last && tile + tile_stride < n_tiles) {        // the activation buffer is dead: fetch the slot's next tile
        if (row == 0) issue_input(tile + tile_stride);
        in_flight = true;
      }

      // ---- epilogue -------------------------------------------------------------------------------
      const float* bias = (sBoff[l] >= 0 && !((spec.bias_in_gemm >> l) & 1)) ? reinterpret_cast<const float*>(wsm + sBoff[l]) : nullptr;
      const int act_l = sAct[l];
      if (spec.pe_stage && l == 0) {
        // f = first 27 accumulator columns; expand to the 150-wide decoder input, in place
        float f[32];
        {
          uint32_t r[32];
          tc05::tmem_ld32_nowait(tmem_lane, r);
          tc05::tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
        }
        float x[160];
#pragma unroll
        for (int i = 0; i < 27; ++i) {
          x[i] = f[i];
          float s1, c1;
          __sincosf(f[i], &s1, &c1);
          const float s2 = 2.f * s1 * c1, c2 = 1.f - 2.f * s1 * s1;   // double-angle: half the SFU work
          x[30 + 2 * i] = s1; x[31 + 2 * i] = s2;
          x[84 + 2 * i] = c1; x[85 + 2 * i] = c2;
        }
#pragma unroll
        for (int i = 0; i < 3; ++i) {
          x[27 + i] = dir[i];
          float s1, c1;
          __sincosf(dir[i], &s1, &c1);
          const float s2 = 2.f * s1 * c1, c2 = 1.f - 2.f * s1 * s1;
          x[138 + 2 * i] = s1; x[139 + 2 * i] = s2;
          x[144 + 2 * i] = c1; x[145 + 2 * i] = c2;
        }
        x[150] = 1.f;                               // ones column: multiplies the bias column of the next layer's weights
#pragma unroll
        for (int i = 151; i < 160; ++i) x[i] = 0.f;
#pragma unroll
        for (int c = 0; c < 20; ++c) store_chunk(act, c, row, x + 8 * c);
      } else {
        // Accumulator columns come out of tensor memory 64 at a time (two 32-column loads in flight, one wait): the
        // loads' latencies overlap, which is what bounds this kernel (one thread walks a whole row of the tile).
        auto finish16 = [&](float* v, int n0) {
          if (bias) {                              // biases sit 16-byte aligned in the blob: four per shared-memory load
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
              const float4 b4 = *reinterpret_cast<const float4*>(bias + n0 + i);
              v[i] += b4.x; v[i + 1] += b4.y; v[i + 2] += b4.z; v[i + 3] += b4.w;
            }
          }
          if (!last && act_l == ACT_RELU) {
            // hidden layer: relu and the bf16 packing are one conversion instruction per pair of columns
            store_chunk_relu(act, (n0 >> 3), row, v);
            store_chunk_relu(act, (n0 >> 3) + 1, row, v + 8);
            return;
          }
          // the activation is uniform per layer: branch once per 16 columns instead of letting the
          // compiler evaluate every transcendental for every element and select
          switch (act_l) {
            case ACT_RELU:
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
              break;
            case ACT_SIGMOID: {
              const int need = last ? spec.out_dim - n0 : 16;       // the output layer is padded to 16 columns
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (i < need) v[i] = __fdividef(1.f, 1.f + __expf(-v[i]));
              break;
            }
            case ACT_TANH:
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = tanhf(v[i]);
              break;
            case ACT_EXP:
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = __expf(v[i]);
              break;
            default: break;
          }
          if (!last) {
            store_chunk(act, (n0 >> 3), row, v);
            store_chunk(act, (n0 >> 3) + 1, row, v + 8);
          } else if (row0 + row < n_rows) {
            float* o = out + (row0 + row) * (long long)out_stride;
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (n0 + i < spec.out_dim) o[n0 + i] = v[i];
          }
        };
        int n0 = 0;
        for (; n0 + 64 <= N; n0 += 64) {
          uint32_t r[64];
          tc05::tmem_ld32_nowait(tmem_lane + n0, r);
          tc05::tmem_ld32_nowait(tmem_lane + n0 + 32, r + 32);
          tc05::tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[16 * q + i]);
            finish16(v, n0 + 16 * q);
          }
        }
        for (; n0 < N; n0 += 16) {
          float v[16];
          tc05::tmem_ld16(tmem_lane + n0, v);
          finish16(v, n0);
        }
        if (!last && sK[l + 1] > N) {
          // the next layer reads more columns than this one produced: a ones column (its weights carry the bias there)
          // followed by zeros
          float fill[8] = {1.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          store_chunk(act, N >> 3, row, fill);
          fill[0] = 0.f;
          for (int c = (N >> 3) + 1; c < (sK[l + 1] >> 3); ++c) store_chunk(act, c, row, fill);
        }
      }
      // TMEM reads and shared-memory writes of this slot are complete before the next MMA / TMA
      tc05::fence_before_sync();
      tc05::fence_async_shared();
      tc05::bar_sync(bar_id, kSlotThreads);
    }
  }

  // a bounded wait gave up with the next tile's copy still in flight: let it land before shared memory is released
  if (in_flight) tc05::mbar_wait(&bar_in[slot], ph_in);
  tc05::fence_before_sync();
  __syncthreads();
  if (tid < 32) tc05::tmem_dealloc(tmem_base_sh, 512);
}

}  // namespace lmb

using namespace lmb;

// xs[s]: [max_rows, widths[s]] bf16 row-major (widths multiples of 8, summing to spec.in_width); a source may
// be a peer GPU's buffer.  out: fp32 [max_rows, out_stride].  status: device int, set non-zero if a
// bounded wait expired.
LMB_API int lmb_fused_mlp_fwd_multi(const void* const* xs, const int* widths, int n_src, const int* count_ptr,
                                    long long max_rows, const void* blob, const MLPSpec* spec, float* out, int out_stride,
                                    int* status, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (n_src < 1 || n_src > kMaxSources) return (int)cudaErrorInvalidValue;
  if (spec->n_layers < 1 || spec->n_layers > kMaxLayers || spec->in_width % 8 || spec->in_width > kMaxK ||
      spec->blob_bytes % 16)
    return (int)cudaErrorInvalidValue;
  for (int l = 0; l < spec->n_layers; ++l)
    if (spec->K[l] % 16 || spec->K[l] > kMaxK || spec->N[l] % 16 || spec->N[l] > kSlotCols || spec->N[l] < 16)
      return (int)cudaErrorInvalidValue;
  MLPInputs inputs;
  inputs.n_src = n_src;
  inputs.n128 = inputs.n64 = 0;
  inputs.x0 = (const __nv_bfloat16*)xs[0];
  int chunk = 0;
  for (int s = 0; s < n_src; ++s) {
    if (widths[s] % 8 || widths[s] <= 0) return (int)cudaErrorInvalidValue;
    inputs.chunk_begin[s] = chunk;
    int rc = encode_input_map(&inputs.map[s], xs[s], widths[s], max_rows);
    if (rc) return rc;
    chunk += widths[s] / 8;
  }
  for (int s = n_src; s <= kMaxSources; ++s) inputs.chunk_begin[s] = chunk;
  if (chunk * 8 != spec->in_width) return (int)cudaErrorInvalidValue;
  // A single source is copied as whole rows into the swizzled layouts (LMB_MLP_WHOLE_ROWS=0 keeps the 8-column chunk
  // copies, which several sources always use): 3 copy instructions and 384 requests per 160-column tile instead of 20
  // and 2560, measured 0.236 ms against 0.298 ms per Mi rows of the colour head.
  static const int whole_rows = getenv("LMB_MLP_WHOLE_ROWS") ? atoi(getenv("LMB_MLP_WHOLE_ROWS")) : 1;
  if (whole_rows && n_src == 1) {
    const int w = spec->in_width, rem = w % 64;
    inputs.n128 = w / 64 + (rem > 32 ? 1 : 0);
    inputs.n64 = (rem > 0 && rem <= 32) ? 1 : 0;
    if (inputs.n128 * 64 + inputs.n64 * 32 < spec->K[0]) return (int)cudaErrorInvalidValue;
    if (inputs.n128) { int rc = encode_swizzled_map(&inputs.map[0], xs[0], w, max_rows, 64); if (rc) return rc; }
    if (inputs.n64) { int rc = encode_swizzled_map(&inputs.map[1], xs[0], w, max_rows, 32); if (rc) return rc; }
  }
  const size_t smem = ((spec->blob_bytes + 1023) & ~1023) + (size_t)kSlots * kActBytes + 1024;
  if (smem > 226 * 1024) return (int)cudaErrorInvalidValue;
  static size_t configured = 0;
  if (smem > configured) {
    LMB_CUDA_TRY(cudaFuncSetAttribute(fused_mlp_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = smem;
  }
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long tiles = (max_rows + kTileRows - 1) / kTileRows;
  const int grid = (int)((tiles + kSlots - 1) / kSlots < sms ? (tiles + kSlots - 1) / kSlots : sms);
  fused_mlp_kernel<<<grid, kSlots * kSlotThreads, smem, stream>>>(inputs, (const unsigned char*)blob, *spec, count_ptr,
                                                                max_rows, out, out_stride, status);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_fused_mlp_fwd(const void* x, const int* count_ptr, long long max_rows, const void* blob,
                              const MLPSpec* spec, float* out, int out_stride, int* status, cudaStream_t stream) {
  const void* xs[1] = {x};
  const int widths[1] = {spec->in_width};
  return lmb_fused_mlp_fwd_multi(xs, widths, 1, count_ptr, max_rows, blob, spec, out, out_stride, status, stream);
}
