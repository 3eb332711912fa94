// All-to-all dispatch / combine over NVLink peer memory for spatial-block (branch) model parallelism.
//
// Every sample is routed to the GPU that owns the spatial block it falls into.  The reference instead
// has every rank of the model-parallel group process the SAME rays, evaluate only its own block and
// exchange the results with variable-length list all-gathers preceded by host syncs
// (landmark/nerf_components/data/samples.py:283-309).  Here:
//   dispatch: a source thread appends its record (payload + source slot) to the owner's inbox segment
//             reserved for that source with a plain peer store; slots come from a local counter, so no
//             remote atomics and no pre-exchange of counts are needed;
//   collect : opens with a device-side barrier folded into its prologue (its first block publishes this rank's
//             per-owner counts and an epoch flag to every peer - "my dispatch is complete" - and all blocks wait
//             for every source's flag), then compacts the P inbox segments;
//   combine : the owner stores each result row straight into the source's output buffer at the sample's slot;
//   result  : opens with the same kind of prologue ("my combine is complete" / wait for every owner) and reads
//             this rank's rows back.
// The backward runs the same hand-over with the roles of payload and result swapped.  No kernel of
// this file is bracketed by a separate barrier launch: the signalling lives in the kernels (peer_sync.cuh).
//
// Buffers of one channel (one kind of query) on every rank, all in peer-mapped memory:
//   inbox  [world][cap][RS] floats, ginbox [world][cap][VS] floats, out [cap][V] floats,
//   incoming int[world] (rows each source sent me), flags unsigned[3][world] (ready / done / grads ready).
// Re-use across calls needs no extra synchronisation: a source dispatches call t+1 only after it has seen every
// owner's "done" flag of call t, which an owner raises after it has read its inbox of call t; an owner writes a
// source's output buffer for call t+1 only after that source's dispatch of call t+1; gradient inboxes are
// written again only after a full forward hand-over, which is ordered after the owner's previous backward.
#include "common.cuh"
#include "peer_sync.cuh"

namespace lmb {

constexpr int kA2AMaxPeers = 8;
constexpr int kA2AMaxRecord = 12;                       // floats: payload up to 11 wide + slot
__host__ __device__ inline int record_stride(int W) { return (W + 1 + 3) & ~3; }
__host__ __device__ inline int grad_stride(int V) { return V == 1 ? 1 : (V + 3) & ~3; }

struct A2APeers {
  void* p[kA2AMaxPeers];
};

// Device-resident state of one channel on this rank (plain local memory, zero-initialised):
// [0] epoch of the "records landed" hand-over, [1] of "results landed", [2] of "gradients landed" (each bumped by the
// last block of the kernel that waited for it), [3..5] the block tickets of those kernels, [8..15] per-owner row counts
// of the dispatch in flight.
constexpr int kStReadyEpoch = 0, kStDoneEpoch = 1, kStGradEpoch = 2, kStTicket = 3, kStCounts = 8, kStWords = 16;
constexpr int kFlagReady = 0, kFlagDone = 1, kFlagGrad = 2;       // rows of the flags array, each `kA2AMaxPeers` words

// payload: [n, W] floats; dst[n]: owner rank or -1.  inbox layout on every rank: [world][cap][RS] floats with the record
// stride RS = W + 1 rounded up to 4 floats, so a record is written and read as whole 16-byte words (a remote 4-byte store
// costs an NVLink packet of its own; the slot index rides in the last used float).
// pos_out[n]: position inside the (dst, src) segment (needed to route gradients back).  Only the first
// *count_ptr rows are sent (device-side count; nullptr: all n).  Slots are claimed once per BLOCK and destination:
// rows are ranked per destination with shared-memory counters, then one global atomic per (block, destination)
// reserves the block's range - 256 times fewer same-address atomics than one per row.
__global__ void __launch_bounds__(256)
a2a_dispatch_kernel(const float* __restrict__ payload, int payload_stride, const int* __restrict__ dst,
                    const float* __restrict__ dst_f, int dst_f_stride, const int* __restrict__ count_ptr, long long n,
                    int W, A2APeers inbox, int src_rank, int world, long long cap, unsigned* __restrict__ state,
                    int* __restrict__ pos_out, int* __restrict__ dst_out, int* overflow) {
  __shared__ int local_count[kA2AMaxPeers], base[kA2AMaxPeers];
  int* counts = reinterpret_cast<int*>(state + kStCounts);
  if (threadIdx.x < kA2AMaxPeers) local_count[threadIdx.x] = 0;
  __syncthreads();
  const long long n_valid = resolve_count(count_ptr, n);
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  int d = -1;
  if (i < n_valid) {
    // the owner comes as an int array or as a float column (the block id the sampler wrote next to the coordinates)
    d = dst ? dst[i] : (int)dst_f[i * dst_f_stride];
    if (d >= world) d = -1;
  }
  if (dst_out && i < n) dst_out[i] = d;
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
  if (pos >= 0) {
    const int RS = record_stride(W);
    float r[kA2AMaxRecord];
#pragma unroll
    for (int k = 0; k < kA2AMaxRecord; ++k) r[k] = k < W ? payload[i * payload_stride + k] : 0.f;
#pragma unroll
    for (int k = 0; k < kA2AMaxRecord; ++k) if (k == W) r[k] = __int_as_float((int)i);
    float4* rec = reinterpret_cast<float4*>(reinterpret_cast<float*>(inbox.p[d]) + ((long long)src_rank * cap + pos) * RS);
#pragma unroll
    for (int q = 0; q < kA2AMaxRecord / 4; ++q)
      if (4 * q < RS) rec[q] = make_float4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
  }
}

// Compact the inbox segments in source order: coords [M, 4] = (payload xyz, block id 0), extra [M, W - 3] = the
// remaining payload columns (may be null), route (src, slot); *total = M = sum of incoming; incoming_saved [world] keeps
// the counts for the backward (the live array is overwritten by the next dispatch of any peer).
__global__ void __launch_bounds__(256)
a2a_collect_kernel(const float* __restrict__ inbox, const int* incoming, A2APeers incoming_peers, PeerFlagPtrs flags,
                   const unsigned* flags_local, unsigned* state, int rank, int world, long long cap, int W,
                   float4* __restrict__ coords, float* __restrict__ extra, int* __restrict__ route_src,
                   int* __restrict__ route_slot, int* __restrict__ total, int* __restrict__ incoming_saved, int* status) {
  const unsigned epoch = state[kStReadyEpoch] + 1u;
  if (blockIdx.x == 0 && (int)threadIdx.x < world) {
    // this rank's dispatch has completed (stream order): hand its per-owner counts to the owners, reset them for the
    // next dispatch; the release store inside publish_and_wait orders the count store before the flag
    int* counts = reinterpret_cast<int*>(state + kStCounts);
    const int c = counts[threadIdx.x];
    reinterpret_cast<int*>(incoming_peers.p[threadIdx.x])[rank] = c < cap ? c : (int)cap;
    counts[threadIdx.x] = 0;
  }
  publish_and_wait(flags, kFlagReady * kA2AMaxPeers, flags_local, rank, world, epoch, kSyncDefaultLimit, status, 200);
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
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) *total = (int)base;
    if ((int)threadIdx.x < world) incoming_saved[threadIdx.x] = incoming[threadIdx.x];
  }
  if (grid_last_block(state + kStTicket + 0) && threadIdx.x == 0) state[kStReadyEpoch] = epoch;
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

// Source side: wait until every owner has delivered, then copy the rows that were sent out of the landing buffer
// (rows that were not sent - no owner, beyond the count, dropped on overflow - read as zero).
__global__ void __launch_bounds__(256)
a2a_result_kernel(const float* out_landing, const int* __restrict__ dst, const int* __restrict__ pos,
                  const int* __restrict__ count_ptr, long long n, int V, PeerFlagPtrs flags, const unsigned* flags_local,
                  unsigned* state, int rank, int world, float* __restrict__ result, int* status) {
  const unsigned epoch = state[kStDoneEpoch] + 1u;       // "my combine is complete" out, "every owner's combine is complete" in
  publish_and_wait(flags, kFlagDone * kA2AMaxPeers, flags_local, rank, world, epoch, kSyncDefaultLimit, status, 300);
  const long long n_valid = resolve_count(count_ptr, n);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const bool sent = i < n_valid && dst[i] >= 0 && dst[i] < world && pos[i] >= 0;
    for (int k = 0; k < V; ++k) result[i * V + k] = sent ? out_landing[i * V + k] : 0.f;
  }
  if (grid_last_block(state + kStTicket + 1) && threadIdx.x == 0) state[kStDoneEpoch] = epoch;
}

// Backward of combine: a source sends d_out[i, :V] to the owner's gradient inbox at (src, pos[i]).
__global__ void __launch_bounds__(256)
a2a_grad_dispatch_kernel(const float* __restrict__ dout, const int* __restrict__ dst, const int* __restrict__ pos,
                         const int* __restrict__ count_ptr, long long n, int V, A2APeers ginbox, int src_rank, int world,
                         long long cap) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < resolve_count(count_ptr, n)) {
    const int d = dst[i], p = pos[i];
    if (d >= 0 && d < world && p >= 0) {
      const int VS = grad_stride(V);
      float* rec = reinterpret_cast<float*>(ginbox.p[d]) + ((long long)src_rank * cap + p) * VS;
      if (V == 1) {
        rec[0] = dout[i];
      } else {
        for (int q = 0; 4 * q < VS; ++q) {                      // whole 16-byte words, zero tail
          float4 v;
          v.x = 4 * q < V ? dout[i * V + 4 * q] : 0.f;         v.y = 4 * q + 1 < V ? dout[i * V + 4 * q + 1] : 0.f;
          v.z = 4 * q + 2 < V ? dout[i * V + 4 * q + 2] : 0.f; v.w = 4 * q + 3 < V ? dout[i * V + 4 * q + 3] : 0.f;
          reinterpret_cast<float4*>(rec)[q] = v;
        }
      }
    }
  }
}

__global__ void __launch_bounds__(256)
a2a_grad_collect_kernel(const float* ginbox, const int* __restrict__ incoming_saved, PeerFlagPtrs flags,
                        const unsigned* flags_local, unsigned* state, int rank, int world, long long cap, int V,
                        float* __restrict__ rows, int* status) {
  const unsigned epoch = state[kStGradEpoch] + 1u;
  publish_and_wait(flags, kFlagGrad * kA2AMaxPeers, flags_local, rank, world, epoch, kSyncDefaultLimit, status, 400);
  long long base = 0;
  for (int s = 0; s < world; ++s) {
    const int c = incoming_saved[s];
    for (long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x; k < c; k += (long long)gridDim.x * blockDim.x) {
      const float* rec = ginbox + ((long long)s * cap + k) * grad_stride(V);
      for (int j = 0; j < V; ++j) rows[(base + k) * V + j] = rec[j];
    }
    base += c;
  }
  if (grid_last_block(state + kStTicket + 2) && threadIdx.x == 0) state[kStGradEpoch] = epoch;
}

}  // namespace lmb

using namespace lmb;

static void fill(A2APeers& dst, const long long* table, int world) {
  for (int i = 0; i < kA2AMaxPeers; ++i) dst.p[i] = i < world ? (void*)table[i] : nullptr;
}
static void fill_flags(PeerFlagPtrs& dst, const long long* table, int world) {
  for (int i = 0; i < kSyncMaxPeers; ++i) dst.p[i] = i < world ? (unsigned*)table[i] : nullptr;
}

// state: this rank's channel state (kStWords zero-initialised words of ordinary device memory).
// *_table: host arrays of `world` peer addresses of the channel's inbox / incoming / flags / out / ginbox regions.
// payload rows are `payload_stride` floats apart (>= W).  The owner of row i is dst[i] (int) or, when dst is null,
// (int)dst_f[i * dst_f_stride]; dst_out (optional) receives it as int for the later kernels of the query.
LMB_API int lmb_a2a_dispatch(const float* payload, int payload_stride, const int* dst, const float* dst_f, int dst_f_stride,
                             const int* count_ptr, long long n, int W, const long long* inbox_table, int rank, int world,
                             long long cap, unsigned* state, int* pos_out, int* dst_out, int* overflow, cudaStream_t stream) {
  if (world > kA2AMaxPeers || W + 1 > kA2AMaxRecord || n <= 0 || payload_stride < W || (dst == nullptr && dst_f == nullptr))
    return (int)cudaErrorInvalidValue;
  A2APeers inbox;
  fill(inbox, inbox_table, world);
  a2a_dispatch_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(payload, payload_stride, dst, dst_f, dst_f_stride, count_ptr, n, W, inbox,
                                                           rank, world, cap, state, pos_out, dst_out, overflow);
  LMB_LAUNCH_CHECK();
  return 0;
}

// coords: [world * cap, 4]; extra: [world * cap, W - 3] or null when W == 3; total: device int; incoming_saved: int[world]
LMB_API int lmb_a2a_collect(const float* inbox, const int* incoming, const long long* incoming_table, const long long* flags_table,
                            const unsigned* flags_local, unsigned* state, int rank, int world, long long cap, int W, float* coords,
                            float* extra, int* route_src, int* route_slot, int* total, int* incoming_saved, int* status,
                            cudaStream_t stream) {
  if (W < 3 || W + 1 > kA2AMaxRecord || (W > 3 && extra == nullptr) || world > kA2AMaxPeers) return (int)cudaErrorInvalidValue;
  A2APeers incoming_peers;
  PeerFlagPtrs flags;
  fill(incoming_peers, incoming_table, world);
  fill_flags(flags, flags_table, world);
  a2a_collect_kernel<<<148 * 4, 256, 0, stream>>>(inbox, incoming, incoming_peers, flags, flags_local, state, rank, world, cap, W,
                                                  (float4*)coords, extra, route_src, route_slot, total, incoming_saved, status);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_combine(const float* values, const int* route_src, const int* route_slot, const int* count_ptr, long long m,
                            int V, const long long* out_table, int world, cudaStream_t stream) {
  if (m <= 0) return (int)cudaErrorInvalidValue;
  A2APeers outs;
  fill(outs, out_table, world);
  const long long want = (m + 255) / 256;            // capped grid: m is the owner-side row capacity
  a2a_combine_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>(values, route_src, route_slot, count_ptr, m, V,
                                                                                 outs);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_result(const float* out_landing, const int* dst, const int* pos, const int* count_ptr, long long n, int V,
                           const long long* flags_table, const unsigned* flags_local, unsigned* state, int rank, int world,
                           float* result, int* status, cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  PeerFlagPtrs flags;
  fill_flags(flags, flags_table, world);
  const long long want = (n + 255) / 256;
  a2a_result_kernel<<<(int)(want < 148 * 16 ? want : 148 * 16), 256, 0, stream>>>(out_landing, dst, pos, count_ptr, n, V, flags,
                                                                                flags_local, state, rank, world, result, status);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_grad_dispatch(const float* dout, const int* dst, const int* pos, const int* count_ptr, long long n, int V,
                                  const long long* ginbox_table, int rank, int world, long long cap, cudaStream_t stream) {
  if (n <= 0) return (int)cudaErrorInvalidValue;
  A2APeers g;
  fill(g, ginbox_table, world);
  a2a_grad_dispatch_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(dout, dst, pos, count_ptr, n, V, g, rank, world, cap);
  LMB_LAUNCH_CHECK();
  return 0;
}

LMB_API int lmb_a2a_grad_collect(const float* ginbox, const int* incoming_saved, const long long* flags_table,
                                 const unsigned* flags_local, unsigned* state, int rank, int world, long long cap, int V, float* rows,
                                 int* status, cudaStream_t stream) {
  PeerFlagPtrs flags;
  fill_flags(flags, flags_table, world);
  a2a_grad_collect_kernel<<<148 * 4, 256, 0, stream>>>(ginbox, incoming_saved, flags, flags_local, state, rank, world, cap, V, rows,
                                                       status);
  LMB_LAUNCH_CHECK();
  return 0;
}
