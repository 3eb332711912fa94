// Fused compute + collective kernels over NVLink peer memory (plain P2P loads / stores).
//
// (1) zero_adam_p2p - data-parallel gradient reduce-scatter + partitioned Adam + parameter all-gather in
//     ONE kernel.  Rank r owns the r-th shard of every flat parameter buffer: it loads that shard of
//     every rank's gradient straight from peer HBM, reduces, applies Adam to its fp32 master shard
//     (moments live only on the owner), stores the updated values into every rank's parameter buffer
//     (and bf16 shadow) and clears the gradients it consumed.  The reference does a bucketed NCCL
//     all-reduce inside DistributedDataParallel followed by a replicated torch.optim.Adam
//     (benchmarks/nerf/gridnerf/gridnerf_trainer.py:120-154).
// (2) composite_merge_p2p - model-parallel rendering: every GPU holds, for every ray, the partial
//     colour / transmittance / depth of the ray segment that crosses ITS spatial blocks plus the
//     segment's entry distance.  Rank r merges the r-th slice of rays: it pulls the P partials of each
//     ray from the peers, orders them by entry distance and alpha-composites them front to back, then
//     stores the finished pixels into the output image of the root (or of every rank).  The reference
//     has no model-parallel rendering merge (its engine only gathers data-parallel ray slices,
//     landmark/render/parallel_module/parallel_module.py:105-135).
// Cross-GPU ordering around both kernels comes from the device-side barrier in symm.cu.
#include "common.cuh"
#include "peer_sync.cuh"

namespace lmb {

constexpr int kMaxPeers = 8;

struct PeerPtrs {
  void* p[kMaxPeers];
};

struct AdamP2PArgs {
  float lr, beta1, beta2, eps, bias1, bias2, grad_scale;
};

// n4: number of float4 elements of the whole flat buffer; shard = [begin4, end4).
// Each thread handles kUnroll float4 per trip and issues all of their peer loads before using any, so
// that enough NVLink requests are in flight to cover the link latency.
constexpr int kAdamUnroll = 4;

__global__ void __launch_bounds__(256)
zero_adam_p2p_kernel(PeerPtrs grads, PeerPtrs params, PeerPtrs shadows, float4* __restrict__ m, float4* __restrict__ v,
                     int world, long long begin4, long long end4, AdamP2PArgs a, int has_shadow) {
  const float step = a.lr / a.bias1;
  const float inv_sqrt_b2 = rsqrtf(a.bias2);
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long base = begin4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; base < end4; base += stride * kAdamUnroll) {
    float4 g[kAdamUnroll], pp[kAdamUnroll], mm[kAdamUnroll], vv[kAdamUnroll];
#pragma unroll
    for (int u = 0; u < kAdamUnroll; ++u) g[u] = zero;
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p) {
      if (p >= world) break;
#pragma unroll
      for (int u = 0; u < kAdamUnroll; ++u) {
        const long long i = base + u * stride;
        if (i < end4) {
          const float4 x = __ldcv(reinterpret_cast<const float4*>(grads.p[p]) + i);   // peer load over NVLink
          g[u].x += x.x; g[u].y += x.y; g[u].z += x.z; g[u].w += x.w;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kAdamUnroll; ++u) {
      const long long i = base + u * stride;
      if (i < end4) {
        pp[u] = reinterpret_cast<float4*>(params.p[0])[i];   // params.p[0] is the local replica
        mm[u] = m[i - begin4];
        vv[u] = v[i - begin4];
      }
    }
#pragma unroll
    for (int u = 0; u < kAdamUnroll; ++u) {
      const long long i = base + u * stride;
      if (i >= end4) continue;
      float* G = &g[u].x; float* P = &pp[u].x; float* M = &mm[u].x; float* V = &vv[u].x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gr = G[k] * a.grad_scale;
        M[k] = a.beta1 * M[k] + (1.f - a.beta1) * gr;
        V[k] = a.beta2 * V[k] + (1.f - a.beta2) * gr * gr;
        P[k] -= step * M[k] / (sqrtf(V[k]) * inv_sqrt_b2 + a.eps);
      }
      m[i - begin4] = mm[u]; v[i - begin4] = vv[u];
      reinterpret_cast<float4*>(grads.p[0])[i] = zero;   // local gradient shard; remote ones are cleared by
                                                         // their owners after the closing barrier
      uint2 sh;
      if (has_shadow) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(pp[u].x, pp[u].y), hi = __floats2bfloat162_rn(pp[u].z, pp[u].w);
        sh.x = *reinterpret_cast<unsigned*>(&lo); sh.y = *reinterpret_cast<unsigned*>(&hi);
      }
#pragma unroll
      for (int p = 0; p < kMaxPeers; ++p) {   // all-gather: push the new values to every rank
        if (p >= world) break;
        reinterpret_cast<float4*>(params.p[p])[i] = pp[u];
        if (has_shadow) reinterpret_cast<uint2*>(shadows.p[p])[i] = sh;
      }
    }
  }
}

// partial layout per ray: 8 floats = r, g, b, T, depth, acc, t_entry, pad
__global__ void __launch_bounds__(256)
composite_merge_p2p_kernel(PeerPtrs partials, PeerPtrs outs, int world, int rank, int root, long long ray_begin,
                           long long ray_end, float bg) {
  const long long r = ray_begin + (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= ray_end) return;
  float4 a[kMaxPeers], b[kMaxPeers];
  int order[kMaxPeers];
#pragma unroll
  for (int p = 0; p < kMaxPeers; ++p) {
    if (p >= world) break;
    const float4* src = reinterpret_cast<const float4*>(partials.p[p]) + 2 * r;
    a[p] = src[0];   // r g b T
    b[p] = src[1];   // depth acc t_entry pad
    order[p] = p;
  }
  // insertion sort of at most 8 segments by entry distance
  for (int i = 1; i < world; ++i) {
    const int k = order[i];
    int j = i - 1;
    while (j >= 0 && b[order[j]].z > b[k].z) { order[j + 1] = order[j]; --j; }
    order[j + 1] = k;
  }
  float T = 1.f, C0 = 0.f, C1 = 0.f, C2 = 0.f, D = 0.f, A = 0.f;
  for (int i = 0; i < world; ++i) {
    const int k = order[i];
    C0 += T * a[k].x; C1 += T * a[k].y; C2 += T * a[k].z;
    D += T * b[k].x; A += T * b[k].y;
    T *= a[k].w;
  }
  const float4 px = make_float4(C0 + T * bg, C1 + T * bg, C2 + T * bg, T);
  const float2 da = make_float2(D, A);
#pragma unroll
  for (int p = 0; p < kMaxPeers; ++p) {
    if (p >= world) break;
    if (root >= 0 && p != root) continue;
    float* o = reinterpret_cast<float*>(outs.p[p]) + 6 * r;
    reinterpret_cast<float2*>(o)[0] = make_float2(px.x, px.y);
    reinterpret_cast<float2*>(o)[1] = make_float2(px.z, px.w);
    reinterpret_cast<float2*>(o)[2] = da;
  }
}

// Small all-reduce over peer memory: every rank has copied its values into its staging buffer; each rank
// sums all staging buffers (plain peer loads, rank order fixed so every rank gets bit-identical sums).
// Used for the gradients of replicated heads (tens of thousands of floats), where a library collective is
// all launch latency and cannot be recorded alongside the peer barriers of the same step.
// The hand-over is a device-side barrier folded into the summing kernel's prologue (peer_sync.cuh): its first block
// raises this rank's epoch flag on every peer ("my staging copy is complete"), all blocks wait for every rank's flag.  Staging is double-buffered by
// epoch parity, so no rank can overwrite a buffer that a slower peer is still summing: a rank stages epoch e+2 only after
// it has summed epoch e+1, for which it needed every peer's flag of e+1, which a peer raises after it summed epoch e.
// state: [0] epoch, [1] block ticket (zero-initialised local words).
__global__ void __launch_bounds__(256)
allreduce_stage_kernel(const float4* __restrict__ in, float4* staging_local, long long n4, long long capacity4,
                       const unsigned* __restrict__ state) {
  const unsigned epoch = state[0] + 1u;                  // bumped by the summing kernel that follows
  float4* dst = staging_local + (long long)(epoch & 1u) * capacity4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) dst[i] = in[i];
}

__global__ void __launch_bounds__(256)
allreduce_small_kernel(PeerPtrs staging, PeerFlagPtrs flags, int rank, int world, long long n4, long long capacity4,
                       unsigned* state, const unsigned* flags_local, float4* __restrict__ out, float scale, int* status) {
  const unsigned epoch = state[0] + 1u;
  publish_and_wait(flags, 0, flags_local, rank, world, epoch, kSyncDefaultLimit, status, 500);
  const long long off = (long long)(epoch & 1u) * capacity4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = reinterpret_cast<const float4*>(staging.p[r])[off + i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    out[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
  }
  if (grid_last_block(state + 1) && threadIdx.x == 0) state[0] = epoch;
}

// ---- fan-out of streamed scene blocks ------------------------------------------------------------------------
// Dynamic loading with several GPUs: every rank reads 1/P of a new block from pinned host memory over its own PCIe
// link, then stores its piece into the same place of every peer's window over NVLink.  The reference has the group
// leader read everything and broadcast it with NCCL (landmark/render/parameter_loader/buffer_manager.py:68-80).
constexpr int kMaxFanoutSegs = 32;
struct FanoutSegs {
  long long off[kMaxFanoutSegs];     // byte offset inside the window, multiple of 16
  long long bytes[kMaxFanoutSegs];   // multiple of 16
};

__global__ void __launch_bounds__(256)
fanout_push_kernel(const char* __restrict__ local, PeerPtrs peers, FanoutSegs segs, int rank, int world) {
  const int s = blockIdx.y;
  const long long n16 = segs.bytes[s] >> 4;
  const uint4* src = reinterpret_cast<const uint4*>(local + segs.off[s]);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = src[i];
    for (int p = 0; p < world; ++p)
      if (p != rank) reinterpret_cast<uint4*>(reinterpret_cast<char*>(peers.p[p]) + segs.off[s])[i] = v;
  }
}

}  // namespace lmb

using namespace lmb;

static void fill_peers(PeerPtrs& dst, const long long* table, int world, int rank_first) {
  // rotate so that entry 0 is the local rank (kernels treat p[0] as "mine" where it matters)
  for (int i = 0; i < kMaxPeers; ++i) dst.p[i] = nullptr;
  for (int i = 0; i < world; ++i) dst.p[i] = (void*)table[(rank_first + i) % world];
}

// grad_table / param_table / shadow_table: host arrays of `world` peer addresses (same byte offset in
// every rank's symmetric buffer).  n must be a multiple of 4 * world.  m, v: local, n / world floats.
LMB_API int lmb_zero_adam_p2p(const long long* grad_table, const long long* param_table, const long long* shadow_table,
                              float* m, float* v, long long n, int rank, int world, float lr, float beta1, float beta2,
                              float eps, int step, float grad_scale, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || n % (4LL * world) != 0) return (int)cudaErrorInvalidValue;
  PeerPtrs g, p, s;
  fill_peers(g, grad_table, world, rank);
  fill_peers(p, param_table, world, rank);
  if (shadow_table) fill_peers(s, shadow_table, world, rank); else for (int i = 0; i < kMaxPeers; ++i) s.p[i] = nullptr;
  AdamP2PArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.grad_scale = grad_scale;
  a.bias1 = 1.f - powf(beta1, (float)step);
  a.bias2 = 1.f - powf(beta2, (float)step);
  const long long shard4 = n / 4 / world;
  const long long begin4 = shard4 * rank, end4 = begin4 + shard4;
  if (shard4 == 0) return 0;
  long long want = (shard4 + 255) / 256;
  const int blocks = (int)(want < 148LL * 8 ? want : 148LL * 8);
  zero_adam_p2p_kernel<<<blocks, 256, 0, stream>>>(g, p, s, (float4*)m, (float4*)v, world, begin4, end4, a,
                                                  shadow_table != nullptr);
  LMB_LAUNCH_CHECK();
  return 0;
}

// After the closing barrier: clear the part of the LOCAL gradient buffer that other ranks own (they have
// finished reading it).  grad_local is this rank's flat gradient buffer of n floats.
LMB_API int lmb_zero_adam_clear_remote_shards(float* grad_local, long long n, int rank, int world, cudaStream_t stream) {
  const long long shard = n / world;
  if (rank > 0) LMB_CUDA_TRY(cudaMemsetAsync(grad_local, 0, (size_t)(shard * rank) * 4, stream));
  if (rank < world - 1)
    LMB_CUDA_TRY(cudaMemsetAsync(grad_local + shard * (rank + 1), 0, (size_t)(shard * (world - 1 - rank)) * 4, stream));
  return 0;
}

// partial_table / out_table: peer addresses of the [R, 8] partial and [R, 6] output buffers.
LMB_API int lmb_composite_merge_p2p(const long long* partial_table, const long long* out_table, long long n_rays, int rank,
                                    int world, int root, float bg, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers) return (int)cudaErrorInvalidValue;
  PeerPtrs part, out;
  for (int i = 0; i < kMaxPeers; ++i) { part.p[i] = nullptr; out.p[i] = nullptr; }
  for (int i = 0; i < world; ++i) { part.p[i] = (void*)partial_table[i]; out.p[i] = (void*)out_table[i]; }
  const long long per = (n_rays + world - 1) / world;
  const long long begin = per * rank, end = begin + per < n_rays ? begin + per : n_rays;
  if (end <= begin) return 0;
  composite_merge_p2p_kernel<<<ceil_div(end - begin, 256), 256, 0, stream>>>(part, out, world, rank, root, begin, end, bg);
  LMB_LAUNCH_CHECK();
  return 0;
}

// in: local fp32 [n] (n a multiple of 4); staging_table / flags_table: per-rank addresses of the staging area (2 x capacity
// floats) and of the flag words (one per source rank); staging_local / flags_local: this rank's; state: 2 zero-initialised
// local words; out: local fp32 [n].  Two launches, no barrier launches around them.
LMB_API int lmb_allreduce_small_p2p(const float* in, const long long* staging_table, const long long* flags_table,
                                    float* staging_local, const unsigned* flags_local, unsigned* state, int rank, int world,
                                    long long n, long long capacity, float* out, float scale, int* status, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n % 4 || capacity % 4 || n > capacity || world > kMaxPeers || world > kSyncMaxPeers) return (int)cudaErrorInvalidValue;
  PeerPtrs st;
  PeerFlagPtrs flags;
  for (int i = 0; i < kMaxPeers; ++i) st.p[i] = i < world ? (void*)staging_table[i] : nullptr;
  for (int i = 0; i < kSyncMaxPeers; ++i) flags.p[i] = i < world ? (unsigned*)flags_table[i] : nullptr;
  const long long n4 = n / 4;
  const int blocks = (int)((n4 + 255) / 256 < 148 * 4 ? (n4 + 255) / 256 : 148 * 4);
  allreduce_stage_kernel<<<blocks, 256, 0, stream>>>((const float4*)in, (float4*)staging_local, n4, capacity / 4, state);
  LMB_LAUNCH_CHECK();
  allreduce_small_kernel<<<blocks, 256, 0, stream>>>(st, flags, rank, world, n4, capacity / 4, state, flags_local, (float4*)out, scale,
                                                     status);
  LMB_LAUNCH_CHECK();
  return 0;
}

// window_table: per-rank base address of the (symmetric) window; offsets/bytes: this rank's pieces, n_segs of them.
// The caller orders the launch after its own host-to-device copies and brackets it with peer barriers.
LMB_API int lmb_fanout_push(const void* local_window, const long long* window_table, const long long* offsets,
                            const long long* bytes, int n_segs, int rank, int world, cudaStream_t stream) {
  if (world > kMaxPeers) return (int)cudaErrorInvalidValue;
  PeerPtrs peers;
  for (int i = 0; i < kMaxPeers; ++i) peers.p[i] = i < world ? (void*)window_table[i] : nullptr;
  for (int base = 0; base < n_segs; base += kMaxFanoutSegs) {
    const int n = n_segs - base < kMaxFanoutSegs ? n_segs - base : kMaxFanoutSegs;
    FanoutSegs segs;
    long long longest = 0;
    for (int k = 0; k < n; ++k) {
      if ((offsets[base + k] | bytes[base + k]) & 15) return (int)cudaErrorInvalidValue;
      segs.off[k] = offsets[base + k]; segs.bytes[k] = bytes[base + k];
      if (bytes[base + k] > longest) longest = bytes[base + k];
    }
    if (longest == 0) continue;
    long long want = ((longest >> 4) + 255) / 256;
    dim3 grid((unsigned)(want < 148 * 2 ? want : 148 * 2), (unsigned)n);
    fanout_push_kernel<<<grid, 256, 0, stream>>>((const char*)local_window, peers, segs, rank, world);
    LMB_LAUNCH_CHECK();
  }
  return 0;
}
