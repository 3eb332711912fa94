// Device-wide exclusive scan and stable LSD radix sort of (64-bit key, 32-bit value) pairs.
//
// Used by the Gaussian rasteriser to order (tile, depth) keys (the reference's rasteriser extension,
// opt_gaussian_rasterization, uses CUB for this; call site benchmarks/nerf/origin_gs/gs_model.py:211-220)
// and by the atomic-free grid backward.  All temporary storage is provided by the caller as one
// scratch buffer, so a call performs no allocation.
//
// Sort pass (8-bit digit): (1) per-block digit histogram, stored digit-major so that one exclusive
// scan over [256][blocks] yields every block's global base per digit; (2) scatter: blocks walk
// their keys in rounds of kThreads, rank equal digits inside a warp with __match_any_sync, order
// warps and rounds through shared-memory counters - stable by construction.
#include "common.cuh"

namespace lmb {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 16;                        // keys per thread per block
constexpr int kSortTile = kSortThreads * kSortItems;  // keys per block
constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;
constexpr int kScanTile = kScanThreads * kScanItems;

// ---- scan -------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t* smem, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    uint32_t y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  if (lane == 31) smem[warp] = x;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = lane < (blockDim.x >> 5) ? smem[lane] : 0;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      uint32_t y = __shfl_up_sync(0xffffffffu, w, d);
      if (lane >= d) w += y;
    }
    smem[lane] = w;
  }
  __syncthreads();
  const uint32_t warp_base = warp ? smem[warp - 1] : 0;
  total = smem[(blockDim.x >> 5) - 1];
  __syncthreads();
  return warp_base + x - v;
}

__global__ void __launch_bounds__(kScanThreads)
scan_tiles_kernel(const uint32_t* in, uint32_t* out, uint32_t* __restrict__ tile_sums, long long n) {
  // `out` may be the same buffer as `in` (the recursion scans the tile sums in place): a thread loads all of its
  // items before it stores any, and it stores only to the positions it loaded, so the two are not marked restrict.
  __shared__ uint32_t sm[32];
  const long long base = (long long)blockIdx.x * kScanTile + threadIdx.x * kScanItems;
  uint32_t v[kScanItems], sum = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) { v[i] = (base + i < n) ? in[base + i] : 0; sum += v[i]; }
  uint32_t total;
  uint32_t excl = block_excl_scan(sum, sm, total);
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) { if (base + i < n) out[base + i] = excl; excl += v[i]; }
  if (threadIdx.x == 0 && tile_sums) tile_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads)
scan_add_kernel(uint32_t* __restrict__ out, const uint32_t* __restrict__ tile_offsets, long long n) {
  const uint32_t off = tile_offsets[blockIdx.x];
  const long long base = (long long)blockIdx.x * kScanTile + threadIdx.x * kScanItems;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) if (base + i < n) out[base + i] += off;
}

// scratch layout for scan of n items: level-1 sums (ceil(n/T)), level-2 sums (ceil(l1/T)), ...
static long long scan_scratch_elems(long long n) {
  long long total = 0;
  while (n > kScanTile) { n = (n + kScanTile - 1) / kScanTile; total += n; }
  return total + 1;
}

static int exclusive_scan(const uint32_t* in, uint32_t* out, long long n, uint32_t* scratch, cudaStream_t stream) {
  const long long tiles = (n + kScanTile - 1) / kScanTile;
  if (tiles <= 1) {
    scan_tiles_kernel<<<1, kScanThreads, 0, stream>>>(in, out, nullptr, n);
    LMB_LAUNCH_CHECK();
    return 0;
  }
  scan_tiles_kernel<<<(int)tiles, kScanThreads, 0, stream>>>(in, out, scratch, n);
  LMB_LAUNCH_CHECK();
  int rc = exclusive_scan(scratch, scratch, tiles, scratch + tiles, stream);
  if (rc) return rc;
  scan_add_kernel<<<(int)tiles, kScanThreads, 0, stream>>>(out, scratch, n);
  LMB_LAUNCH_CHECK();
  return 0;
}

// ---- radix sort ----------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSortThreads)
radix_hist_kernel(const uint64_t* __restrict__ keys, const int* __restrict__ count_ptr, long long max_n, int shift,
                  uint32_t* __restrict__ hist, int n_blocks) {
  __shared__ uint32_t h[256];
  h[threadIdx.x] = 0;
  __syncthreads();
  const long long n = resolve_count(count_ptr, max_n);
  const long long base = (long long)blockIdx.x * kSortTile;
  for (int i = threadIdx.x; i < kSortTile; i += kSortThreads) {
    const long long idx = base + i;
    if (idx < n) atomicAdd(&h[(keys[idx] >> shift) & 0xFF], 1u);
  }
  __syncthreads();
  hist[(long long)threadIdx.x * n_blocks + blockIdx.x] = h[threadIdx.x];
}

__global__ void __launch_bounds__(kSortThreads)
radix_scatter_kernel(const uint64_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                     uint64_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, const int* __restrict__ count_ptr,
                     long long max_n, int shift, const uint32_t* __restrict__ offsets, int n_blocks) {
  __shared__ uint32_t running[256];                   // next free slot of each digit for this block
  __shared__ uint32_t warp_cnt[kSortThreads / 32][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  running[threadIdx.x] = offsets[(long long)threadIdx.x * n_blocks + blockIdx.x];
  const long long n = resolve_count(count_ptr, max_n);
  const long long base = (long long)blockIdx.x * kSortTile;
  for (int r = 0; r < kSortItems; ++r) {
    for (int w = 0; w < kSortThreads / 32; ++w) warp_cnt[w][threadIdx.x] = 0;
    __syncthreads();
    const long long idx = base + (long long)r * kSortThreads + threadIdx.x;
    const bool valid = idx < n;
    uint64_t key = 0;
    uint32_t val = 0, digit = 0xFFFFFFFFu;
    if (valid) { key = keys_in[idx]; val = vals_in[idx]; digit = (uint32_t)(key >> shift) & 0xFF; }
    const uint32_t peers = __match_any_sync(0xffffffffu, digit);
    const uint32_t rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (valid && rank_in_warp == 0) warp_cnt[warp][digit] = __popc(peers);
    __syncthreads();
    // thread d turns the per-warp counts of digit d into exclusive offsets and advances running[d]
    {
      uint32_t acc = running[threadIdx.x];
      for (int w = 0; w < kSortThreads / 32; ++w) {
        const uint32_t c = warp_cnt[w][threadIdx.x];
        warp_cnt[w][threadIdx.x] = acc;
        acc += c;
      }
      running[threadIdx.x] = acc;
    }
    __syncthreads();
    if (valid) {
      const uint32_t pos = warp_cnt[warp][digit] + rank_in_warp;
      keys_out[pos] = key;
      vals_out[pos] = val;
    }
    __syncthreads();
  }
}

}  // namespace lmb

using namespace lmb;

LMB_API long long lmb_scan_scratch_bytes(long long n) { return scan_scratch_elems(n) * 4; }

LMB_API int lmb_exclusive_scan_u32(const uint32_t* in, uint32_t* out, long long n, void* scratch, cudaStream_t stream) {
  if (n <= 0) return 0;
  return exclusive_scan(in, out, n, (uint32_t*)scratch, stream);
}

// Bytes of scratch needed to sort up to max_n pairs: the alternate key/value buffers, the digit
// histogram and the scan workspace.
LMB_API long long lmb_radix_sort_scratch_bytes(long long max_n) {
  const long long blocks = (max_n + kSortTile - 1) / kSortTile;
  const long long hist = 256 * blocks;
  long long bytes = max_n * 8 + max_n * 4;            // alternate buffers
  bytes = (bytes + 255) & ~255LL;
  bytes += hist * 4;
  bytes = (bytes + 255) & ~255LL;
  bytes += scan_scratch_elems(hist) * 4 + 256;
  return bytes;
}

// Sorts (keys, vals) in place (the result lands back in the input arrays) on bits [begin_bit, end_bit).
// (end_bit - begin_bit) is rounded up to a multiple of 8; an odd number of passes costs one copy back.
LMB_API int lmb_radix_sort_pairs(uint64_t* keys, uint32_t* vals, const int* count_ptr, long long max_n, int begin_bit,
                                 int end_bit, void* scratch, cudaStream_t stream) {
  if (max_n <= 0) return 0;
  const long long blocks = (max_n + kSortTile - 1) / kSortTile;
  const long long hist_n = 256 * blocks;
  unsigned char* p = (unsigned char*)scratch;
  uint64_t* keys_alt = (uint64_t*)p; p += max_n * 8;
  uint32_t* vals_alt = (uint32_t*)p; p += max_n * 4;
  p = (unsigned char*)(((uintptr_t)p + 255) & ~(uintptr_t)255);
  uint32_t* hist = (uint32_t*)p; p += hist_n * 4;
  p = (unsigned char*)(((uintptr_t)p + 255) & ~(uintptr_t)255);
  uint32_t* scan_ws = (uint32_t*)p;
  uint64_t* kin = keys; uint32_t* vin = vals; uint64_t* kout = keys_alt; uint32_t* vout = vals_alt;
  int passes = 0;
  for (int shift = begin_bit; shift < end_bit; shift += 8, ++passes) {
    radix_hist_kernel<<<(int)blocks, kSortThreads, 0, stream>>>(kin, count_ptr, max_n, shift, hist, (int)blocks);
    LMB_LAUNCH_CHECK();
    int rc = exclusive_scan(hist, hist, hist_n, scan_ws, stream);
    if (rc) return rc;
    radix_scatter_kernel<<<(int)blocks, kSortThreads, 0, stream>>>(kin, vin, kout, vout, count_ptr, max_n, shift, hist, (int)blocks);
    LMB_LAUNCH_CHECK();
    uint64_t* tk = kin; kin = kout; kout = tk;
    uint32_t* tv = vin; vin = vout; vout = tv;
  }
  if (passes & 1) {
    LMB_CUDA_TRY(cudaMemcpyAsync(keys, kin, max_n * 8, cudaMemcpyDeviceToDevice, stream));
    LMB_CUDA_TRY(cudaMemcpyAsync(vals, vin, max_n * 4, cudaMemcpyDeviceToDevice, stream));
  }
  return 0;
}

// ---- allocation-free scan entry point (declared in lmb_noalloc.h) ---------------------------------------
#include <mutex>
#include "lmb_noalloc.h"

namespace {

// Workspace of the allocation-free scan.  It lives in every CUDA context that loads this library
// (LMB_NOALLOC_SCAN_SCRATCH_BYTES per GPU, until the process exits) and is shared by all calls.
static __device__ __align__(256) unsigned char g_noalloc_scan_scratch[LMB_NOALLOC_SCAN_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mutex;
void* g_noalloc_scratch_ptr[kMaxDevices] = {nullptr};

// Resolve the device address of the workspace for the current device.  The array's name is only a
// host-side handle in host code; the address a kernel can use has to come from the runtime.
int noalloc_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return LMB_NOALLOC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scan_scratch);
    if (e != cudaSuccess) return (int)e;
    g_noalloc_scratch_ptr[dev] = p;
  }
  *out = g_noalloc_scratch_ptr[dev];
  return 0;
}

}  // namespace

LMB_API int lmb_exclusive_scan_u32_noalloc(const uint32_t* in, uint32_t* out, long long n, cudaStream_t stream) {
  if (n < 0 || in == nullptr || out == nullptr) return LMB_NOALLOC_ERR_ARGUMENT;
  if (n == 0) return 0;
  if (n > LMB_NOALLOC_SCAN_MAX_ELEMS || scan_scratch_elems(n) * 4 > (long long)LMB_NOALLOC_SCAN_SCRATCH_BYTES)
    return LMB_NOALLOC_ERR_TOO_LARGE;
  void* scratch = nullptr;
  const int rc = noalloc_scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  // Every workspace word that is read (per-tile sums of each level) is written earlier in the same
  // call, so nothing has to be cleared even though the array keeps the previous call's contents.
  return exclusive_scan(in, out, n, (uint32_t*)scratch, stream);
}
