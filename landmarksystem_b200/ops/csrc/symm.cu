// Peer-memory plumbing for the fused compute+collective kernels: symmetric allocations exchanged through
// CUDA IPC handles, and a device-side barrier built from release/acquire flags in peer memory.
//
// The reference moves every tensor between GPUs with NCCL calls from the host
// (landmark/communicator/collective.py:13-155); here kernels read and write peer HBM directly over
// NVLink, so a "collective" is ordinary loads/stores inside the compute kernel plus this barrier.
// Every wait is bounded: after ~1 s of SM clocks the kernel records an error status and returns, so
// a peer that never arrives can not hang the GPU.
#include "common.cuh"

namespace lmb {

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// flags_local[p] is written by peer p.  peer_flags[p] points at peer p's flag array.
// One block: thread p signals peer p then waits for peer p's signal.
// The epoch lives in device memory (*epoch_dev counts the barriers this rank has passed), so the same
// launch can be replayed from a CUDA graph; every rank runs the same sequence of barriers.
__global__ void barrier_kernel(unsigned* flags_local, unsigned* const* peer_flags, int rank, int world, unsigned* epoch_dev,
                               long long limit_cycles, int* status) {
  const int p = threadIdx.x;
  const unsigned epoch = *epoch_dev + 1u;
  __syncthreads();
  if (p == 0) *epoch_dev = epoch;
  if (p >= world) return;
  __threadfence_system();
  st_release_sys(peer_flags[p] + rank, epoch);
  const long long t0 = clock64();
  while ((int)(ld_acquire_sys(flags_local + p) - epoch) < 0) {
    if (clock64() - t0 > limit_cycles) { atomicExch(status, 100 + p); return; }
  }
}

}  // namespace lmb

using namespace lmb;

LMB_API int lmb_symm_alloc(long long bytes, void** out) {
  void* p = nullptr;
  LMB_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
  LMB_CUDA_TRY(cudaMemset(p, 0, (size_t)bytes));
  *out = p;
  return 0;
}

LMB_API int lmb_symm_free(void* p) {
  LMB_CUDA_TRY(cudaFree(p));
  return 0;
}

LMB_API int lmb_ipc_get_handle(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  LMB_CUDA_TRY(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, sizeof(h));
  return 0;
}

LMB_API int lmb_ipc_open(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* p = nullptr;
  LMB_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return 0;
}

LMB_API int lmb_ipc_close(void* p) {
  LMB_CUDA_TRY(cudaIpcCloseMemHandle(p));
  return 0;
}

// Device-side barrier over `world` ranks on `stream`.  status: device int, set to 100 + p if the wait for peer p
// gave up after `limit_cycles` SM clocks (<= 0: the default of about one second).
LMB_API int lmb_peer_barrier(unsigned* flags_local, unsigned* const* peer_flags, int rank, int world, unsigned* epoch_dev,
                             int* status, long long limit_cycles, cudaStream_t stream) {
  if (world > 32) return (int)cudaErrorInvalidValue;
  if (limit_cycles <= 0) limit_cycles = 2000000000LL;
  barrier_kernel<<<1, 32, 0, stream>>>(flags_local, peer_flags, rank, world, epoch_dev, limit_cycles, status);
  LMB_LAUNCH_CHECK();
  return 0;
}
