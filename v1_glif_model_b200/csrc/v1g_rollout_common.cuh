// Helpers shared by the forward and backward persistent rollout kernels.
#pragma once

#include "v1g_internal.h"

struct V1GRolloutPlan {
  int chunk;    // neurons per block
  int chunkP;   // chunk rounded up to 32 (stride of the on-chip state planes)
  int grid;     // blocks
  size_t state_bytes;
  size_t fixed_bytes;
};

size_t v1g_plan_rollout(const V1GHandle* h, int B, int per_item_floats, int per_item_bytes,
                        int fixed_per_neuron_bytes, V1GRolloutPlan* p);

__device__ __forceinline__ unsigned long long v1g_ld_acquire(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Grid-wide barrier on a monotonically increasing counter.  Every block adds 1 and waits until
// the counter reaches `target` (= number of barriers passed so far x grid size).  The wait is
// bounded: after `spin_limit` polls the block records V1G_DEV_BARRIER_TIMEOUT in the device
// status word and every block that sees a non-zero status leaves its time loop, so a lost block
// can never hang the GPU.  Requires a cooperative launch (all blocks co-resident).
__device__ __forceinline__ bool v1g_grid_barrier(unsigned long long* bar, unsigned long long target,
                                                 long long spin_limit, int32_t* status,
                                                 int* s_abort) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(bar, 1ULL);
    long long spins = 0;
    bool ok = true;
    while (v1g_ld_acquire(bar) < target) {
      if (++spins > spin_limit) {
        ok = false;
        break;
      }
    }
    if (!ok) atomicExch(status, V1G_DEV_BARRIER_TIMEOUT);
    if (*((volatile int32_t*)status) != V1G_DEV_OK) ok = false;
    *s_abort = ok ? 0 : 1;
    __threadfence();
  }
  __syncthreads();
  return *s_abort == 0;
}

__device__ __forceinline__ unsigned long long v1g_warp_sum(unsigned long long v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return v;
}
