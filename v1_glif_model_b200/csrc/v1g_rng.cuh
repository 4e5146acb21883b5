// Counter-based random numbers shared by the sampling kernels and the LGN event compaction.
#pragma once

#include <algorithm>

#include "v1g_internal.h"

#define V1G_POISSON_TABLE 32
#define V1G_RNG_STREAM_BKG 0x42u  // fourth counter word: keeps the two samplers on disjoint counters
#define V1G_RNG_STREAM_LGN 0x4cu

// Philox-4x32 with 10 rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011):
// a bijection of the 128-bit counter under a 64-bit key.
__host__ __device__ __forceinline__ uint4 v1g_philox4x32(uint4 ctr, uint2 key) {
  const unsigned M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = (unsigned long long)M0 * ctr.x, p1 = (unsigned long long)M1 * ctr.z;
    const unsigned hi0 = (unsigned)(p0 >> 32), lo0 = (unsigned)p0, hi1 = (unsigned)(p1 >> 32), lo1 = (unsigned)p1;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}

// uniform in [0, 1) with 24 random bits (exact in float32)
__host__ __device__ __forceinline__ float v1g_u01(unsigned w) { return (float)(w >> 8) * (1.0f / 16777216.0f); }

// One Bernoulli draw of LGN unit c of trial b at step t: true with probability
// 1 - exp(-rate / 1000), rate in Hz, dt = 1 ms (stim_dataset.py:182-193).
__device__ __forceinline__ bool v1g_lgn_spike(float rate_hz, int b, int t, int c, unsigned key0, unsigned key1) {
  const uint4 r = v1g_philox4x32(make_uint4((unsigned)(c >> 2), (unsigned)t, (unsigned)b, V1G_RNG_STREAM_LGN),
                                 make_uint2(key0, key1));
  const unsigned w = (c & 3) == 0 ? r.x : (c & 3) == 1 ? r.y : (c & 3) == 2 ? r.z : r.w;
  const float p = -expm1f(-rate_hz * 0.001f);
  return v1g_u01(w) < p;
}

// Poisson counts of the background nodes for T steps from (seed, replica, step) into out[B,T,n_bkg];
// the first step is step0 + step0_dev[0] (step0_dev may be NULL).
int v1g_sample_bkg_internal(V1GHandle* h, int B, int T, const int32_t* step0_dev, int step0, int32_t* out,
                            cudaStream_t st);
// noise_step[b] += T for every trial (nullable pointer: nothing to do)
int v1g_advance_noise_step(V1GHandle* h, int32_t* noise_step, int B, int T, cudaStream_t st);
