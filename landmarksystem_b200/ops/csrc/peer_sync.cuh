// Signalling between kernels that run on different GPUs, folded into the kernels themselves.
//
// A producer kernel stores into peer memory.  The kernel that follows it on the same stream - the consumer of what the
// PEERS produced - opens with `publish_and_wait`: its first block publishes an epoch number into a flag word on every
// peer (release, system scope: "my producer has finished"), and all of its blocks wait until the flag words of all
// ranks have reached that epoch (acquire, system scope) before they read the peers' data.  Compared with a separate
// barrier kernel between producer and consumer this saves the launch and hides the consumer's launch latency.  The reference synchronises the same hand-over with host-side list
// all-gathers (landmark/nerf_components/data/samples.py:283-309).
//
// Every wait is bounded: after `limit` SM clocks the waiting thread records `error_base + peer` in a status word and
// the kernel carries on (its results are then wrong, which the host learns from the status word), so a peer that
// never arrives cannot hang the GPU.
#pragma once
#include "common.cuh"

namespace lmb {

constexpr int kSyncMaxPeers = 8;
constexpr long long kSyncDefaultLimit = 2000000000LL;     // about one second of SM clocks

struct PeerFlagPtrs {
  unsigned* p[kSyncMaxPeers];       // p[r]: the flag array (one word per source rank) in rank r's memory
};

__device__ __forceinline__ void st_release_sys_u32(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Bookkeeping helper: returns true in exactly one block of the grid - the last one to get here.  No memory ordering is
// implied (a plain ticket), so it is cheap; use it for device-side counters that must change only after every block
// of the launch has read them.  `ticket` is a zero-initialised device word; it is reset for the next launch.
__device__ __forceinline__ bool grid_last_block(unsigned* ticket) {
  __shared__ int last_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned total = gridDim.x * gridDim.y * gridDim.z;
    const unsigned t = atomicAdd(ticket, 1u);
    last_flag = (t == total - 1);
    if (last_flag) *ticket = 0;
  }
  __syncthreads();
  return last_flag != 0;
}

// Prologue of a consumer kernel, called by all threads of every block.  Block 0 first tells every peer that this
// rank's PRODUCER (the previous kernel on this rank's stream, complete by stream order, its peer stores included) is
// done, by publishing `epoch` into the peers' flag words for this rank; then every block waits until all ranks'
// flag words here have reached `epoch`.  A device-side barrier, but without a launch of its own and with the
// consumer's launch latency hidden behind the wait.  A per-block system fence in the producer would achieve the same
// without relying on the kernel boundary, and costs tens of microseconds on kernels with thousands of blocks.
__device__ __forceinline__ void publish_and_wait(const PeerFlagPtrs& flags, int flag_offset, const unsigned* flags_local,
                                                 int rank, int world, unsigned epoch, long long limit, int* status,
                                                 int error_base) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && (int)threadIdx.x < world) {
    __threadfence_system();
    st_release_sys_u32(flags.p[threadIdx.x] + flag_offset + rank, epoch);
  }
  if ((int)threadIdx.x < world) {
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys_u32(flags_local + flag_offset + threadIdx.x) - epoch) < 0) {
      if (clock64() - t0 > limit) {
        if (status) atomicExch(status, error_base + (int)threadIdx.x);
        break;
      }
    }
  }
  __syncthreads();
}

}  // namespace lmb
