// All-to-all dispatch / combine over NVLink peer memory for spatial-block (branch) model parallelism.
//
// Every sample is routed to the GPU that owns the spatial block it falls into.  The reference instead
// has every rank of the model-parallel group process the SAME rays, evaluate only its own block and
// exchange the results with variable-length list all-gathers preceded by host syncs
// (landmark/nerf_components/data/samples.py:283-309).  Here:
//   dispatch: a source thread appends its record (payload + source slot) to the owner's inbox segment
//             reserved for that source with a plain peer store; slots come from a local counter, so no
//             remote atomics and no pre-exchange of counts are needed;
//   collect : the owner compacts the P inbox segments (their counts arrive with the barrier);
//   combine : the owner stores each result row straight into the source's output buffer at the
//             sample's slot - the "scatter back" costs no kernel on the source.
// The same three kernels run the backward with the roles of payload and result swapped.
#include "common.cuh"

namespace lmb {

constexpr int kA2AMaxPeers = 8;
constexpr int kA2AMaxRecord = 12;                       // floats: payload up to 11 wide + slot
__host__ __device__ inline int record_stride(int W) { return (W + 1 + 3) & ~3; }
__host__ __device__ inline int grad_stride(int V) { return V == 1 ? 1 : (V + 3) & ~3; }

struct A2APeers {
  void* p[kA2AMaxPeers];
};

// payload: [n, W] floats; dst[n]: owner rank or -1.  inbox layout on every rank: [world][cap][RS] floats with the record
// stride RS = W + 1 rounded up to 4 floats, so a record is written and read as whole 16-byte words (a remote 4-byte store
// costs an NVLink packet of its own; the slot index rides in the last used float).
// pos_out[n]: position inside the (dst, src) segment (needed to route gradients back).  Only the first
// *count_ptr rows are sent (device-side count; nullptr: all n).  Slots are claimed once per BLOCK and destination:
// rows are ranked per destination with shared-memory counters, then one global atomic per (block, destination)
// reserves the block's range - 256 times fewer same-address atomics than one per row.
__global__ void __launch_bounds__(256)
a2a_dispatch_kernel(const float* __restrict__ payload, const int* __restrict__ dst, const int* __restrict__ count_ptr, long long n,
                    int W, A2APeers inbox, int src_rank, int world, long long cap, int* __restrict__ counts,
                    int* __restrict__ pos_out, int* overflow) {
  __shared__ int local_count[kA2AMaxPeers], base[kA2AMaxPeers];
  if (threadIdx.x < kA2AMaxPeers) local_count[threadIdx.x] = 0;
  __syncthreads();
  const long long n_valid = resolve_count(count_ptr, n);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int d = -1;
  if (i < n_valid) { d = dst[i]; if (d >= world) d = -1; }
  int local = 0;
  if (d >= 0) local = atomicAdd(&local_count[d], 1);
  __syncthreads();
  if (threadIdx.x < world && local_count[threadIdx.x] > 0)
    base[threadIdx.x] = atomicAdd(&counts[threadIdx.x], local_count[threadIdx.x]);
  __syncthreads();
  int pos = -1;
  if (d >= 0) {
    pos = base[d] + local;
    if (pos >= cap) { pos = -1; atomicExch(overflow, 1); }
  }
  if (i < n) pos_out[i] = pos;
  if (pos < 0) return;
  const int RS = record_stride(W);
  float r[kA2AMaxRecord];
#pragma unroll
  for (int k = 0; k < kA2AMaxRecord; ++k) r[k] = k < W ? payload[i * W + k] : 0.f;
#pragma unroll
  for (int k = 0; k < kA2AMaxRecord; ++k) if (k == W) r[k] = __int_as_float((int)i);
  float4* rec = reinterpret_cast<float4*>(reinterpret_cast<float*>(inbox.p[d]) + ((long long)src_rank * cap + pos) * RS);
#pragma unroll
  for (int q = 0; q < kA2AMaxRecord / 4; ++q)
    if (4 * q < RS) rec[q] = make_float4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
}

// counts of this rank are copied into every peer's incoming[src_rank]
__global__ void a2a_publish_kernel(const int* __restrict__ counts, A2APeers incoming, int src_rank, int world, long long cap) {
  const int d = threadIdx.x;
  if (d >= world) return;
  const int c = counts[d];
  reinterpret_cast<int*>(incoming.p[d])[src_rank] = c < cap ? c : (int)cap;
}

// Compact the inbox segments in source order: coords [M, 4] = (payload xyz, block id 0), extra [M, W - 3] = the
// remaining payload columns (may be null), route (src, slot); *total = M = sum of incoming.
__global__ void __launch_bounds__(256)
a2a_collect_kernel(const float* __restrict__ inbox, const int* __restrict__ incoming, int world, long long cap, int W,
                   float4* __restrict__ coords, float* __restrict__ extra, int* __restrict__ route_src,
                   int* __restrict__ route_slot, int* __restrict__ total) {
  long long base = 0;
  const int E = W - 3, RS = record_stride(W);
  for (int s = 0; s < world; ++s) {
    const int c = incoming[s];
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < c; k += (long long)gridDim.x * blockDim.x) {
      const float4* rec4 = reinterpret_cast<const float4*>(inbox + ((long long)s * cap + k) * RS);
      float r[kA2AMaxRecord];
#pragma unroll
      for (int q = 0; q < kA2AMaxRecord / 4; ++q)
        if (4 * q < RS) { const float4 v = rec4[q]; r[4 * q] = v.x; r[4 * q + 1] = v.y; r[4 * q + 2] = v.z; r[4 * q + 3] = v.w; }
      coords[base + k] = make_float4(r[0], r[1], r[2], 0.f);
      int slot = 0;
#pragma unroll
      for (int j = 3; j < kA2AMaxRecord; ++j) {
        if (j < W) extra[(base + k) * E + (j - 3)] = r[j];
        if (j == W) slot = __float_as_int(r[j]);
      }
      route_src[base + k] = s;
      route_slot[base + k] = slot;
    }
    base += c;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) *total = (int)base;
}

// values: [M, V]; written to outs[src] + slot * V
__global__ void __launch_bounds__(256)
a2a_combine_kernel(const float* __restrict__ values, const int* __restrict__ route_src, const int* __restrict__ route_slot,
                   const int* __restrict__ count_ptr, long long m, int V, A2APeers outs) {
  const long long n = resolve_count(count_ptr, m);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float* o = reinterpret_cast<float*>(outs.p[route_src[i]]) + (long long)route_slot[i] * V;
    for (int k = 0; k < V; ++k) o[k] = values[i * V + k];
  }
}

// Backward of combine: a source sends d_out[i, :V] to the owner's gradient inbox at (src, pos[i]).
__global__ void __launch_bounds__(256)
a2a_grad_dispatch_kernel(const float* __restrict__ dout, const int* __restrict__ dst, const int* __restrict__ pos,
                         const int* __restrict__ count_ptr, long long n, int V, A2APeers ginbox, int src_rank, long long cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= resolve_count(count_ptr, n)) return;
  const int d = dst[i], p = pos[i];
  if (d < 0 || p < 0) return;
  const int VS = grad_stride(V);
  float* rec = reinterpret_cast<float*>(ginbox.p[d]) + ((long long)src_rank * cap + p) * VS;
  if (V == 1) { rec[0] = dout[i]; return; }
  for (int q = 0; 4 * q < VS; ++q) {                      // whole 16-byte words, zero tail
    float4 v;
    v.x = 4 * q < V ? dout[i * V + 4 * q] : 0.f;         v.y = 4 * q + 1 < V ? dout[i * V + 4 * q + 1] : 0.f;
    v.z = 4 * q + 2 < V ? dout[i * V + 4 * q + 2] : 0.f; v.w = 4 * q + 3 < V ? dout[i * V + 4 * q + 3] : 0.f;
    reinterpret_cast<float4*>(rec)[q] = v;
  }
}

__global__ void __launch_bounds__(256)
a2a_grad_collect_kernel(const float* __restrict__ ginbox, const int* __restrict__ incoming, int world, long long cap, int V,
                        float* __restrict__ rows) {
  long long base = 0;
  for (int s = 0; s < world; ++s) {
    const int c = incoming[s];
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < c; k += (long long)gridDim.x * blockDim.x) {
      const float* rec = ginbox + ((long long)s * cap + k) * grad_stride(V);
      for (int j = 0; j < V; ++j) rows[(base + k) * V + j] = rec[j];
    }
    base += c;
  }
}

}  // namespace lmb

using namespace lmb;

static void fill(A2APeers& dst, const long long* table, int world) {
  for (int i = 0; i < kA2AMaxPeers; ++i) dst.p[i] = i < world ? (void*)table[i] : nullptr;
}

LMB_API int lmb_a2a_dispatch(const float* payload, const int* dst, const int* count_ptr, long long n, int W,
                             const long long* inbox_table, const long long* incoming_table, int rank, int world, long long cap,
                             int* counts, int* pos_out, int* overflow, cudaStream_t stream) {
  if (world > kA2AMaxPeers || W + 1 > kA2AMaxRecord) return (int)cudaErrorInvalidValue;
  A2APeers inbox, incoming;
  fill(inbox, inbox_table, world);
  fill(incoming, incoming_table, world);
  LMB_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * world, stream));
  if (n > 0)
    a2a_dispatch_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(payload, dst, count_ptr, n, W, inbox, rank, world, cap, counts,
                                                             pos_out, overflow);
  a2a_publish_kernel<<<1, 32, 0, stream>>>(counts, incoming, rank, world, cap);
  LMB_LAUNCH_CHECK();
  return 0;
}

// coords: [world * cap, 4]; extra: [world * cap, W - 3] or null when W == 3; total: device int
LMB_API int lmb_a2a_collect(const float* inbox, const int* incoming, int world, long long cap, int W, float* coords, float* extra,
                            int* route_src, int* route_slot, int* total, cudaStream_t stream) {
  if (W < 3 || W + 1 > kA2AMaxRecord || (W > 3 && extra == nullptr)) return (int)cudaErrorInvalidValue;
  a2a_collect_kernel<<<148 * 4, 256, 0, stream>>>(inbox, incoming, world, cap, W, (float4*)coords, extra, route_src, route_slot,
                                                  total);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_combine(const float* values, const int* route_src, const int* route_slot, const int* count_ptr, long long m,
                            int V, const long long* out_table, int world, cudaStream_t stream) {
  if (m <= 0) return 0;
  A2APeers outs;
  fill(outs, out_table, world);
  const long long want = (m + 255) / 256;            // capped grid: m is the owner-side row capacity
  a2a_combine_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>(values, route_src, route_slot, count_ptr, m, V, outs);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_grad_dispatch(const float* dout, const int* dst, const int* pos, const int* count_ptr, long long n, int V,
                                  const long long* ginbox_table, int rank, int world, long long cap, cudaStream_t stream) {
  if (n <= 0) return 0;
  A2APeers g;
  fill(g, ginbox_table, world);
  a2a_grad_dispatch_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(dout, dst, pos, count_ptr, n, V, g, rank, cap);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_grad_collect(const float* ginbox, const int* incoming, int world, long long cap, int V, float* rows,
                                 cudaStream_t stream) {
  a2a_grad_collect_kernel<<<148 * 4, 256, 0, stream>>>(ginbox, incoming, world, cap, V, rows);
  LMB_LAUNCH_CHECK();
  return 0;
}
