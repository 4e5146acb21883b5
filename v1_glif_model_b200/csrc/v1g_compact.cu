// Ordered spike compaction: the device equivalent of tf.where(x > 0) (models.py:128, 826, 890).
//
// Three launches: (1) per-segment counts, (2) one-block exclusive scan of the counts,
// (3) per-segment ordered fill with warp ballots + prefix sums.  The output order is exactly
// row-major (row, col), or (t, b, col) for the time-major LGN list of the fused rollout, and is
// bit-for-bit reproducible (no atomics decide a position).
#include "v1g_rng.cuh"

namespace {

// where the flags come from: an array (positive entries), or LGN firing rates from which the spike
// of (trial, step, unit) is drawn on the fly - the draw is a pure function of its coordinates, so
// the counting and the filling pass see the same flags
template <typename T>
struct ArraySource {
  const T* x;
  int64_t n_cols;
  __device__ __forceinline__ bool operator()(int row, int64_t c) const { return x[(int64_t)row * n_cols + c] > (T)0; }
};
struct RateSource {
  V1GRateSource s;
  int64_t n_cols;
  int T;  // rows are (trial, step) = (row / T, row % T)
  __device__ __forceinline__ bool operator()(int row, int64_t c) const {
    const int b = row / T, t = row - b * T;
    const float rate = s.rates[(int64_t)b * s.batch_stride + (int64_t)t * n_cols + c];
    return v1g_lgn_spike(rate, b, t, (int)c, s.key0, s.key1);
  }
};

// segment id in OUTPUT order for memory row `row`
__device__ __forceinline__ int64_t out_segment(int row, int seg, int nseg, int n_rows, int tmT) {
  if (tmT > 0) {
    const int B = n_rows / tmT;
    const int b = row / tmT, t = row - b * tmT;
    return ((int64_t)t * B + b) * nseg + seg;
  }
  return (int64_t)row * nseg + seg;
}

template <typename SRC>
__global__ void __launch_bounds__(256) count_kernel(const SRC src, int n_rows,
                                                    int64_t n_cols, int nseg, int tmT,
                                                    int32_t* __restrict__ counts) {
  const int64_t blk = blockIdx.x;
  const int row = (int)(blk / nseg), seg = (int)(blk - (int64_t)row * nseg);
  const int64_t c0 = (int64_t)seg * V1G_SEG;
  const int64_t c1 = min(c0 + (int64_t)V1G_SEG, n_cols);
  int cnt = 0;
  for (int64_t c = c0 + threadIdx.x; c < c1; c += blockDim.x) cnt += src(row, c) ? 1 : 0;
  __shared__ int wsum[8];
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_down_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    int s = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) s += wsum[w];
    counts[out_segment(row, seg, nseg, n_rows, tmT)] = s;
  }
}

// In-place exclusive scan of counts[0..m) by one block; counts[m] = total; *total_out = total.
__global__ void __launch_bounds__(1024) scan_kernel(int32_t* __restrict__ counts, int64_t m,
                                                    int32_t* __restrict__ total_out) {
  const int tid = threadIdx.x, nt = blockDim.x;
  const int64_t per = (m + nt - 1) / nt;
  const int64_t i0 = min((int64_t)tid * per, m), i1 = min(i0 + per, m);
  int s = 0;
  for (int64_t i = i0; i < i1; ++i) s += counts[i];
  // block exclusive scan of s
  __shared__ int wtot[32];
  int inc = s;
  for (int o = 1; o < 32; o <<= 1) {
    int v = __shfl_up_sync(0xffffffffu, inc, o);
    if ((tid & 31) >= o) inc += v;
  }
  if ((tid & 31) == 31) wtot[tid >> 5] = inc;
  __syncthreads();
  if (tid < 32) {
    int v = (tid < (nt >> 5)) ? wtot[tid] : 0;
    int iv = v;
    for (int o = 1; o < 32; o <<= 1) {
      int u = __shfl_up_sync(0xffffffffu, iv, o);
      if (tid >= o) iv += u;
    }
    wtot[tid] = iv - v;  // exclusive warp base
  }
  __syncthreads();
  int run = wtot[tid >> 5] + inc - s;
  for (int64_t i = i0; i < i1; ++i) {
    const int c = counts[i];
    counts[i] = run;
    run += c;
  }
  if (tid == nt - 1) {
    counts[m] = run;
    if (total_out) *total_out = run;
  }
}

template <typename SRC, int KIND>
__global__ void __launch_bounds__(256) fill_kernel(const SRC src, int n_rows,
                                                   int64_t n_cols, int nseg, int tmT,
                                                   const int32_t* __restrict__ offsets,
                                                   void* __restrict__ out, int64_t cap) {
  const int64_t blk = blockIdx.x;
  const int row = (int)(blk / nseg), seg = (int)(blk - (int64_t)row * nseg);
  const int64_t c0 = (int64_t)seg * V1G_SEG;
  const int64_t c1 = min(c0 + (int64_t)V1G_SEG, n_cols);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __shared__ int wcnt[8];
  int64_t base = offsets[out_segment(row, seg, nseg, n_rows, tmT)];
  const int b = (tmT > 0) ? row / tmT : row;
  for (int64_t cb = c0; cb < c1; cb += blockDim.x) {
    const int64_t c = cb + threadIdx.x;
    const bool f = (c < c1) && src(row, c);
    const unsigned bal = __ballot_sync(0xffffffffu, f);
    if (lane == 0) wcnt[warp] = __popc(bal);
    __syncthreads();
    int wbase = 0, tot = 0;
    for (int w = 0; w < nw; ++w) {
      const int cw = wcnt[w];
      if (w < warp) wbase += cw;
      tot += cw;
    }
    if (f) {
      const int64_t idx = base + wbase + __popc(bal & ((1u << lane) - 1u));
      if (idx < cap) {
        if (KIND == V1G_COMPACT_F32_COORDS) {
          int64_t* o = (int64_t*)out;
          o[2 * idx] = row;
          o[2 * idx + 1] = c;
        } else {
          ((uint32_t*)out)[idx] = ((uint32_t)b << 24) | (uint32_t)c;
        }
      }
    }
    base += tot;
    __syncthreads();
  }
}

}  // namespace

int v1g_compact_count_scan(V1GHandle* h, int kind, const void* x, int n_rows, int64_t n_cols,
                           int time_major_T, int32_t* offsets, int64_t* n_segments_out,
                           cudaStream_t st) {
  const int nseg = (int)((n_cols + V1G_SEG - 1) / V1G_SEG);
  const int64_t m = (int64_t)n_rows * nseg;
  if (m > 0x7fffffffLL) return v1g_fail(h, V1G_ERANGE, "compaction input too large");
  if (n_segments_out) *n_segments_out = m;
  if (m > 0) {
    if (kind == V1G_COMPACT_F32_COORDS)
      count_kernel<<<(unsigned)m, 256, 0, st>>>(ArraySource<float>{(const float*)x, n_cols}, n_rows, n_cols, nseg,
                                                time_major_T, offsets);
    else if (kind == V1G_COMPACT_U8_PACKED)
      count_kernel<<<(unsigned)m, 256, 0, st>>>(ArraySource<uint8_t>{(const uint8_t*)x, n_cols}, n_rows, n_cols,
                                                nseg, time_major_T, offsets);
    else
      count_kernel<<<(unsigned)m, 256, 0, st>>>(RateSource{*(const V1GRateSource*)x, n_cols, time_major_T}, n_rows,
                                                n_cols, nseg, time_major_T, offsets);
  }
  scan_kernel<<<1, 1024, 0, st>>>(offsets, m, h->d_count);
  v1g_count_launches(m > 0 ? 2 : 1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

int v1g_compact_fill(V1GHandle* h, int kind, const void* x, int n_rows, int64_t n_cols,
                     int time_major_T, const int32_t* offsets, void* out, int64_t cap,
                     cudaStream_t st) {
  const int nseg = (int)((n_cols + V1G_SEG - 1) / V1G_SEG);
  const int64_t m = (int64_t)n_rows * nseg;
  if (m == 0) return V1G_OK;
  if (kind == V1G_COMPACT_F32_COORDS)
    fill_kernel<ArraySource<float>, V1G_COMPACT_F32_COORDS><<<(unsigned)m, 256, 0, st>>>(
        ArraySource<float>{(const float*)x, n_cols}, n_rows, n_cols, nseg, time_major_T, offsets, out, cap);
  else if (kind == V1G_COMPACT_U8_PACKED)
    fill_kernel<ArraySource<uint8_t>, V1G_COMPACT_U8_PACKED><<<(unsigned)m, 256, 0, st>>>(
        ArraySource<uint8_t>{(const uint8_t*)x, n_cols}, n_rows, n_cols, nseg, time_major_T, offsets, out, cap);
  else
    fill_kernel<RateSource, V1G_COMPACT_U8_PACKED><<<(unsigned)m, 256, 0, st>>>(
        RateSource{*(const V1GRateSource*)x, n_cols, time_major_T}, n_rows, n_cols, nseg, time_major_T, offsets,
        out, cap);
  v1g_count_launches(1);
  V1G_CUDA(h, cudaGetLastError());
  return V1G_OK;
}

extern "C" int v1g_compact_spikes(V1GHandle* h, const float* x, int32_t n_rows, int64_t n_cols,
                                  int64_t* coords, int64_t cap, int32_t* count, void* stream) {
  if (!h) return V1G_EINVAL;
  if (n_rows < 0 || n_cols < 0 || cap < 0 || (!x && n_rows * n_cols > 0) || (!coords && cap > 0))
    return v1g_fail(h, V1G_EINVAL, "v1g_compact_spikes: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int nseg = (int)((n_cols + V1G_SEG - 1) / V1G_SEG);
  int rc = v1g_reserve(h, &h->seg_counts, &h->seg_cap, (int64_t)n_rows * nseg + 1);
  if (rc) return rc;
  if ((rc = v1g_compact_count_scan(h, V1G_COMPACT_F32_COORDS, x, n_rows, n_cols, 0, h->seg_counts,
                                   nullptr, st)))
    return rc;
  if ((rc = v1g_compact_fill(h, V1G_COMPACT_F32_COORDS, x, n_rows, n_cols, 0, h->seg_counts, coords,
                             cap, st)))
    return rc;
  if (count)
    V1G_CUDA(h, cudaMemcpyAsync(count, h->d_count, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
  return V1G_OK;
}

// ------------------------------------------------------------------------------------------
// Compaction without any allocation
// ------------------------------------------------------------------------------------------
// v1g_compact_spikes keeps its per-segment counters in a buffer that the handle obtains from
// cudaMalloc.  Some hosts of this code must not do that: an op kernel inside TensorFlow or
// PyTorch is expected to take all device memory from the framework's own allocator (a raw
// cudaMalloc escapes its accounting and stalls every stream of the device while it runs), and a
// caller that only holds a fixed memory budget handed to it at start-up has nothing to allocate
// from.  For them the counters live in the fixed array below, which is part of the library image:
// every GPU on which the library is loaded sets aside 256 KiB for it until the process exits.
#define V1G_NOALLOC_MAX_SEGMENTS 65536
static __device__ __align__(256) int32_t g_noalloc_counters[V1G_NOALLOC_MAX_SEGMENTS + 2];

// In host code the name above is only a handle for the runtime, not something a kernel can be
// given; the device address is looked up once per device and remembered here.
#define V1G_NOALLOC_MAX_DEVICES 64
static int32_t* g_noalloc_counters_dev[V1G_NOALLOC_MAX_DEVICES];

extern "C" int v1g_compact_spikes_noalloc(const float* x, int32_t n_rows, int64_t n_cols,
                                          int64_t* coords, int64_t cap, int32_t* count,
                                          void* stream) {
  if (n_rows < 0 || n_cols < 0 || cap < 0 || (!x && (int64_t)n_rows * n_cols > 0) ||
      (!coords && cap > 0)) {
    v1g_set_global_error("v1g_compact_spikes_noalloc: bad argument");
    return V1G_EINVAL;
  }
  const int64_t nseg = (n_cols + V1G_SEG - 1) / V1G_SEG;
  const int64_t m = (int64_t)n_rows * nseg;
  if (m > V1G_NOALLOC_MAX_SEGMENTS) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "v1g_compact_spikes_noalloc: %lld segments of %d columns exceed the fixed scratch of "
             "%d segments (n_rows * ceil(n_cols / %d) must stay within it)",
             (long long)m, V1G_SEG, V1G_NOALLOC_MAX_SEGMENTS, V1G_SEG);
    v1g_set_global_error(msg);
    return V1G_ERANGE;
  }
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= V1G_NOALLOC_MAX_DEVICES) {
    v1g_set_global_error("v1g_compact_spikes_noalloc: no usable current CUDA device");
    return V1G_ECUDA;
  }
  if (!g_noalloc_counters_dev[dev]) {
    // first call on this device (it is the current one): resolve the array's device address
    int32_t* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, g_noalloc_counters);
    if (e != cudaSuccess || !p) {
      v1g_set_global_error(cudaGetErrorString(e));
      return V1G_ECUDA;
    }
    g_noalloc_counters_dev[dev] = p;
  }
  int32_t* counters = g_noalloc_counters_dev[dev];
  cudaStream_t st = (cudaStream_t)stream;
  const int nseg_i = (int)nseg;
  // every counter the later passes read is written by the count pass of this same call, so the
  // values left by the previous call never need clearing
  if (m > 0)
    count_kernel<<<(unsigned)m, 256, 0, st>>>(ArraySource<float>{x, n_cols}, n_rows, n_cols, nseg_i, 0, counters);
  scan_kernel<<<1, 1024, 0, st>>>(counters, m, count);
  if (m > 0)
    fill_kernel<ArraySource<float>, V1G_COMPACT_F32_COORDS><<<(unsigned)m, 256, 0, st>>>(
        ArraySource<float>{x, n_cols}, n_rows, n_cols, nseg_i, 0, counters, coords, cap);
  v1g_count_launches(m > 0 ? 3 : 1);
  if (cudaGetLastError() != cudaSuccess) {
    v1g_set_global_error("v1g_compact_spikes_noalloc: kernel launch failed");
    return V1G_ECUDA;
  }
  return V1G_OK;
}
