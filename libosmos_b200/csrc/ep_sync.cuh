// Flags between GPUs, for the kernels of the expert-parallel step: a sender's data is followed by a release of a step
// number into a word in the consumer's memory; the consumer's kernels acquire that word (a bounded wait) before they
// read. Plain loads and stores at system scope only: nothing here waits on a kernel of the same GPU, and nothing is
// multicast.
#pragma once
#include "common.cuh"

namespace osmos {

constexpr uint64_t kFlagWaitNs = 2000ull * 1000 * 1000;  // a peer never takes 2 s: past that the wait gives up

__device__ __forceinline__ uint64_t flag_clock_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// true once *flag has reached `step` (acquire - at system scope, or the device's where the one writer is this GPU:
// `alone`); false when the limit ran out first
__device__ __forceinline__ bool flag_wait(const uint32_t* flag, uint32_t step, bool alone) {
  const uint64_t t0 = flag_clock_ns();
  for (;;) {
    uint32_t v;
    if (alone) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    else asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t) (v - step) >= 0) return true;
    if (flag_clock_ns() - t0 > kFlagWaitNs) return false;
    __nanosleep(64);
  }
}

// every rank's exchange buffer as this process maps it (this rank's own among them)
struct EpPeers {
  uint8_t* base[16];
};

// The flags after the data. Every thread of every block calls it when its stores are done: the block meets, one thread
// fences the block's stores at system scope (they are ordered before the barrier, the barrier before the fence: one
// fence a block does what one a thread would, at a few hundredths of the cost) and counts the block in, and the block
// that finds all the others counted writes `step` into its flag word in every rank's buffer (release, system scope),
// optionally stores the step into *bump, and zeroes the counter.
__device__ __forceinline__ void publish_step(const EpPeers& peers, uint64_t flags_off, uint32_t rank, uint32_t n_ranks,
                                             uint32_t step, uint32_t* counter, uint32_t* bump) {
  __shared__ bool s_last;
  __syncthreads();
  // (a rank alone stores into its own GPU's memory only: the fences need not reach past the device)
  if (threadIdx.x == 0) {
    if (n_ranks > 1) __threadfence_system();
    else __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x * gridDim.y - 1;
  }
  __syncthreads();
  if (!s_last) return;
  if (n_ranks > 1) __threadfence_system();  // (the other blocks' counts were seen: their stores before these flags)
  else __threadfence();
  if (threadIdx.x < n_ranks) {
    uint32_t* f = (uint32_t*) (peers.base[threadIdx.x] + flags_off) + rank;
    if (n_ranks > 1) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(step) : "memory");
    else asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(f), "r"(step) : "memory");
  }
  if (threadIdx.x == 0) {
    if (bump) *bump = step;
    *counter = 0;
  }
}

}  // namespace osmos
