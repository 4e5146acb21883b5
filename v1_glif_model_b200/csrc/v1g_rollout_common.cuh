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

// Lagged synchronisation uses one counter per phase, rotating over V1G_PHASES cache lines.  A
// single running sum would not do: with blocks allowed to run ahead, fast blocks could push the
// sum past a target while a slow block has not arrived yet.  Counter p % V1G_PHASES receives one
// arrival per block for phase p, so after phase p it holds (p / V1G_PHASES + 1) * grid.
#define V1G_PHASES 8
#define V1G_PHASE_STRIDE 16  // u64 per counter: one 128-byte line each
#define V1G_BARRIER_BYTES (V1G_PHASES * V1G_PHASE_STRIDE * sizeof(unsigned long long))
__device__ __forceinline__ unsigned long long* v1g_phase_counter(unsigned long long* base, int p) {
  return base + (p % V1G_PHASES) * V1G_PHASE_STRIDE;
}
__device__ __forceinline__ unsigned long long v1g_phase_target(int p, unsigned long long grid) {
  return (unsigned long long)(p / V1G_PHASES + 1) * grid;
}

// One block's arrival at the lagged barrier: release-increment of the counter.  Call from one
// thread after a __syncthreads() that follows the block's last write of the phase.
__device__ __forceinline__ void v1g_arrive(unsigned long long* bar) {
  asm volatile("red.release.gpu.global.add.u64 [%0], 1;" ::"l"(bar) : "memory");
}

// Bounded wait until the counter reaches `target`; returns the last value read.  On timeout the
// device status word is set and the value returned is below the target.
__device__ __forceinline__ unsigned long long v1g_wait(unsigned long long* bar,
                                                       unsigned long long target,
                                                       long long spin_limit, int32_t* status) {
  unsigned long long v = v1g_ld_acquire(bar);
  long long spins = 0;
  while (v < target) {
    if (++spins > spin_limit || *((volatile int32_t*)status) != V1G_DEV_OK) {
      atomicExch(status, V1G_DEV_BARRIER_TIMEOUT);
      return v;
    }
    v = v1g_ld_acquire(bar);
  }
  return v;
}

__device__ __forceinline__ unsigned long long v1g_warp_sum(unsigned long long v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  return v;
}
