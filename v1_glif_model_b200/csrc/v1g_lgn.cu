// LGN front end on the device: movie -> firing rates of the LGN units, the step upstream of the
// cell's input (lgn_model/lgn.py:481-528 with its helpers :54-96).
//
// Reference pipeline per spatial-size class: conv2d of every frame with the class's Gaussian filter
// (padding SAME), division by the same convolution of a frame of ones (its "bmtk_compat" edge
// normalisation), bilinear sampling of the filtered frames at each unit's (x, y) and at the
// position of its non-dominant subfield; then per unit a causal temporal filter over the samples
// (depthwise convolution after front padding), x amplitude + spontaneous rate, rectification, and
// dominant + is_composite * non-dominant.
//
// Here the spatial part is folded into ONE stencil per (unit, subfield), built once when the
// tables are set: the four bilinear corners of the filtered frame are the same movie patch seen
// through four shifted copies of the filter, each divided by its own edge normaliser, so
//     response[t, u] = sum over a (k+1) x (k+1) patch of E[u][dy][dx] * movie[t, y0+dy, x0+dx]
// with taps outside the frame dropped (they are the zero padding; their weights are stored as 0 and
// the coordinates clamped, so the inner loop has no branch).  Stencils are sorted by side and stored
// in groups of 32, one per lane of a warp, tap-major (weight of tap p of lane l at [p][l]), so a warp
// reads one 128-byte line per tap and its lanes run the same trip count; inside a side they are
// ordered so that the lanes of a group fall on different shared-memory banks.  A thread block takes two
// frames, interleaved pixel by pixel, into shared memory (two 120 x 240 frames are 225 KB) and
// evaluates every stencil on both from there: the movie is read from HBM once, a weight fetched from
// L2 serves two frames, and one 8-byte shared-memory load brings both pixels.  The temporal filter
// keeps a sliding window per thread: TT outputs of one unit per thread reuse every loaded sample and
// kernel value TT times.
#include <math.h>

#include <algorithm>
#include <vector>

#include "v1g_internal.h"

struct V1GLgn {
  int n_units = 0, height = 0, width = 0, len_dom = 0, len_non_dom = 0;
  int device = 0, n_sms = 0, smem_optin = 0;
  // stencils of the dominant [0, U) and non-dominant [U, 2U) subfields, sorted by side, 32 per group
  int n_groups = 0;
  int2* st_grp = nullptr;      // [n_groups] = (first tap of the group in st_w / 32, side)
  int4* st_slot = nullptr;     // [n_groups * 32] = (y0, x0, subfield * U + unit or -1 for an empty lane, 0)
  float* st_w = nullptr;       // per group [side * side][32]
  float *k_dom = nullptr, *k_non_dom = nullptr;  // [len][U]
  float *amp = nullptr, *non_dom_amp = nullptr, *composite = nullptr, *spont = nullptr;
  float* spatial = nullptr;    // [2][T][U] scratch, grown on demand
  int64_t spatial_cap = 0;
  std::string err;
};

namespace {

int lgn_fail(V1GLgn* l, int code, const char* msg) {
  if (l) l->err = msg;
  v1g_set_global_error(msg);
  return code;
}

#define LGN_CUDA(l, call)                                                        \
  do {                                                                           \
    cudaError_t e_ = (call);                                                     \
    if (e_ != cudaSuccess) return lgn_fail(l, V1G_ECUDA, cudaGetErrorString(e_)); \
  } while (0)

template <typename T>
int lgn_upload(V1GLgn* l, T** dst, const T* src, size_t n) {
  LGN_CUDA(l, cudaMalloc((void**)dst, std::max<size_t>(n, 1) * sizeof(T)));
  if (n) LGN_CUDA(l, cudaMemcpy(*dst, src, n * sizeof(T), cudaMemcpyHostToDevice));
  return V1G_OK;
}

// one block per F consecutive frames: they go to shared memory interleaved ([pixel][F]) and every
// stencil group is evaluated from there, one group per warp at a time; out[s][t][u].  With F == 1 and
// IN_SMEM false (frames larger than shared memory) the pixels are read from global memory.
constexpr int TB = 8;
template <int F, bool IN_SMEM>
__global__ void __launch_bounds__(1024) lgn_spatial_kernel(const float* __restrict__ movie, int T, int H, int W, int U,
                                                          int n_groups, const int2* __restrict__ st_grp,
                                                          const int4* __restrict__ st_slot,
                                                          const float* __restrict__ st_w, float* __restrict__ out) {
  extern __shared__ float frame_s[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
  const int HW = H * W;
  for (int t0 = blockIdx.x * F; t0 < T; t0 += gridDim.x * F) {
    const int nf = min(F, T - t0);
    const float* frame = movie + (int64_t)t0 * HW;
    if (IN_SMEM) {
      __syncthreads();
      for (int i = threadIdx.x; i < HW; i += blockDim.x) {
#pragma unroll
        for (int f = 0; f < F; ++f) frame_s[i * F + f] = f < nf ? frame[(int64_t)f * HW + i] : 0.f;
      }
      __syncthreads();
    }
    for (int g = warp; g < n_groups; g += n_warps) {
      const int2 gd = st_grp[g];
      const int4 sl = st_slot[g * 32 + lane];
      const int side = gd.y;
      const float* w = st_w + (int64_t)gd.x * 32 + lane;
      float acc[F];
#pragma unroll
      for (int f = 0; f < F; ++f) acc[f] = 0.f;
      // the taps of the patch in row-major order, TB at a time so that TB weight loads are in flight;
      // the table pads every group to a multiple of TB taps with zero weights (their clamped
      // coordinates stay inside the frame)
      const int taps = (side * side + TB - 1) / TB * TB;
      int dy = 0, dx = 0;
      for (int p = 0; p < taps; p += TB) {
        float wv[TB];
#pragma unroll
        for (int j = 0; j < TB; ++j) wv[j] = w[(p + j) * 32];
#pragma unroll
        for (int j = 0; j < TB; ++j) {
          const int px = min(max(sl.x + dy, 0), H - 1) * W + min(max(sl.y + dx, 0), W - 1);
          if (F == 2) {
            const float2 v = IN_SMEM ? *reinterpret_cast<const float2*>(frame_s + 2 * px)
                                     : *reinterpret_cast<const float2*>(frame + 2 * px);
            acc[0] += wv[j] * v.x;
            acc[F - 1] += wv[j] * v.y;
          } else {
            acc[0] += wv[j] * (IN_SMEM ? frame_s[px] : frame[px]);
          }
          if (++dx == side) { dx = 0; ++dy; }
        }
      }
      if (sl.z >= 0) {
        const int sub = sl.z >= U ? 1 : 0, u = sl.z - sub * U;
#pragma unroll
        for (int f = 0; f < F; ++f)
          if (f < nf) out[((int64_t)sub * T + t0 + f) * U + u] = acc[f];
      }
    }
  }
}

// rates[t][u] = relu(amp * f_dom + spont) + composite * relu(nd_amp * f_nd + spont), f = causal filter
// of the unit's samples: f[t] = sum_j K[j] * s[t - (L - 1) + j] with s = 0 before the movie starts.
// A thread owns TT consecutive outputs of one unit and walks the taps TT at a time over a window of
// 2 TT samples held in registers: 2 TT loads feed TT * TT multiply-adds.
constexpr int TT = 8;
__global__ void __launch_bounds__(256) lgn_temporal_kernel(const float* __restrict__ spatial, int T, int U,
                                                           const float* __restrict__ k_dom, int len_dom,
                                                           const float* __restrict__ k_nd, int len_nd,
                                                           const float* __restrict__ amp,
                                                           const float* __restrict__ nd_amp,
                                                           const float* __restrict__ composite,
                                                           const float* __restrict__ spont, float* __restrict__ rates) {
  const int u = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = blockIdx.y * TT;
  if (u >= U) return;
  float f[2][TT];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const float* kern = (s ? k_nd : k_dom) + u;
    const int L = s ? len_nd : len_dom;
    const float* smp = spatial + (int64_t)s * T * U + u;
    auto sample = [&](int q) { return q >= 0 && q < T ? smp[(int64_t)q * U] : 0.f; };
#pragma unroll
    for (int i = 0; i < TT; ++i) f[s][i] = 0.f;
    // output i, tap j reads sample t0 + i - (L - 1) + j; win[i + jj] is that sample for tap j0 + jj
    float win[2 * TT];
    const int q0 = t0 - (L - 1);
#pragma unroll
    for (int i = 0; i < TT; ++i) win[i] = sample(q0 + i);
    for (int j0 = 0; j0 < L; j0 += TT) {
      float kv[TT];
#pragma unroll
      for (int jj = 0; jj < TT; ++jj) {
        kv[jj] = j0 + jj < L ? kern[(int64_t)(j0 + jj) * U] : 0.f;
        win[TT + jj] = sample(q0 + j0 + TT + jj);
      }
#pragma unroll
      for (int jj = 0; jj < TT; ++jj)
#pragma unroll
        for (int i = 0; i < TT; ++i) f[s][i] += kv[jj] * win[i + jj];
#pragma unroll
      for (int i = 0; i < TT; ++i) win[i] = win[TT + i];
    }
  }
  const float a = amp[u], an = nd_amp[u], c = composite[u], sp = spont[u];
#pragma unroll
  for (int i = 0; i < TT; ++i) {
    const int t = t0 + i;
    if (t >= T) break;
    const float d = f[0][i] * a + sp, n = f[1][i] * an + sp;
    rates[(int64_t)t * U + u] = (d >= 0.f ? d : 0.f) + c * (n >= 0.f ? n : 0.f);
  }
}

}  // namespace

extern "C" int v1g_lgn_create(const V1GLgnTables* tb, V1GLgn** out) {
  if (!tb || !out) return lgn_fail(nullptr, V1G_EINVAL, "v1g_lgn_create: null argument");
  *out = nullptr;
  if (tb->n_units <= 0 || tb->height <= 0 || tb->width <= 0 || tb->n_classes <= 0 || tb->len_dom <= 0 ||
      tb->len_non_dom <= 0 || !tb->x || !tb->y || !tb->non_dominant_x || !tb->non_dominant_y || !tb->unit_class ||
      !tb->filter_sizes || !tb->filters || !tb->dom_temporal_kernels || !tb->non_dom_temporal_kernels ||
      !tb->amplitude || !tb->non_dom_amplitude || !tb->is_composite || !tb->spontaneous_firing_rates)
    return lgn_fail(nullptr, V1G_EINVAL, "v1g_lgn_create: bad tables");
  const int U = tb->n_units, H = tb->height, W = tb->width;
  std::vector<int64_t> f_off((size_t)tb->n_classes + 1, 0);
  for (int c = 0; c < tb->n_classes; ++c) {
    const int k = tb->filter_sizes[c];
    if (k <= 0 || (k & 1) == 0) return lgn_fail(nullptr, V1G_EINVAL, "v1g_lgn_create: filter sizes must be odd");
    f_off[c + 1] = f_off[c] + (int64_t)k * k;
  }
  // edge normaliser of a class at a pixel: the sum of the filter taps that fall inside the frame
  auto norm_at = [&](int c, int y, int x) {
    const int k = tb->filter_sizes[c], r = k / 2;
    const float* g = tb->filters + f_off[c];
    double s = 0.0;
    for (int dy = 0; dy < k; ++dy)
      for (int dx = 0; dx < k; ++dx) {
        const int yy = y + dy - r, xx = x + dx - r;
        if (yy >= 0 && yy < H && xx >= 0 && xx < W) s += g[dy * k + dx];
      }
    return s;
  };
  struct Stencil { int y0, x0, side; std::vector<float> w; };
  std::vector<Stencil> sts((size_t)2 * U);
  for (int su = 0; su < 2 * U; ++su) {
    const int s = su >= U, u = su - s * U;
    const int c = tb->unit_class[u];
    if (c < 0 || c >= tb->n_classes) return lgn_fail(nullptr, V1G_EINVAL, "v1g_lgn_create: unit class out of range");
    const float x = s ? tb->non_dominant_x[u] : tb->x[u], y = s ? tb->non_dominant_y[u] : tb->y[u];
    if (!(x >= 0.f && x <= (float)(W - 1) && y >= 0.f && y <= (float)(H - 1)))
      return lgn_fail(nullptr, V1G_EINVAL, "v1g_lgn_create: unit position outside the frame");
    const int k = tb->filter_sizes[c], r = k / 2, side = k + 1;
    const float* g = tb->filters + f_off[c];
    const int xf = (int)floorf(x), yf = (int)floorf(y), xc = (int)ceilf(x), yc = (int)ceilf(y);
    const float fx = x - floorf(x), fy = y - floorf(y);
    // corners in the reference's order (select_spatial, lgn.py:67-96) with their bilinear weights
    const int cy[4] = {yf, yc, yf, yc}, cx[4] = {xf, xf, xc, xc};
    const float cw[4] = {(1.f - fx) * (1.f - fy), (1.f - fx) * fy, fx * (1.f - fy), fx * fy};
    std::vector<double> e((size_t)side * side, 0.0);
    for (int q = 0; q < 4; ++q) {
      if (cw[q] == 0.f) continue;
      const double scale = (tb->bmtk_compat ? 1.0 / norm_at(c, cy[q], cx[q]) : 1.0) * (double)cw[q];
      const int oy = cy[q] - yf, ox = cx[q] - xf;  // 0 or 1: shift of this corner's filter inside the patch
      for (int dy = 0; dy < k; ++dy)
        for (int dx = 0; dx < k; ++dx) e[(size_t)(dy + oy) * side + dx + ox] += scale * (double)g[dy * k + dx];
    }
    Stencil& st = sts[su];
    st.y0 = yf - r; st.x0 = xf - r; st.side = side;
    st.w.resize(e.size());
    for (int dy = 0; dy < side; ++dy)
      for (int dx = 0; dx < side; ++dx) {
        const int yy = st.y0 + dy, xx = st.x0 + dx;
        const bool inside = yy >= 0 && yy < H && xx >= 0 && xx < W;   // outside: the frame's zero padding
        st.w[(size_t)dy * side + dx] = inside ? (float)e[(size_t)dy * side + dx] : 0.f;
      }
  }
  std::vector<int> order((size_t)2 * U);
  for (int i = 0; i < 2 * U; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return sts[a].side < sts[b].side; });
  // Bank conflicts.  The 32 lanes of a group read the same tap (dy, dx) of 32 different patches, so the
  // shared-memory bank of a lane is fixed by its patch corner: (y0 * W + x0) modulo M, M = 16 pixel
  // pairs when two frames are interleaved (a half warp per wavefront), 32 pixels with one frame.
  // Within a run of equal side the stencils are therefore dealt out round-robin over the M residues,
  // so that (almost) every M consecutive lanes hit M different banks: an 8-byte load then takes
  // about 2 wavefronts instead of the 6 that randomly placed patches take (5.7 -> 4.1 ms per 1000
  // frames of 17,400 units).  Measured on top of it and slower: a branch for groups whose patches
  // all lie inside the frame (no clamping, tap offsets from a table per side; 4.8 ms, the groups
  // that cross the edge then cluster), and a warp per stencil with its lanes on consecutive taps
  // (12.5 ms: one stencil's dependent loads at a time per warp).
  {
    cudaDeviceProp prop0;
    int dev0 = 0;
    if (cudaGetDevice(&dev0) != cudaSuccess || cudaGetDeviceProperties(&prop0, dev0) != cudaSuccess)
      return lgn_fail(nullptr, V1G_ECUDA, "v1g_lgn_create: no CUDA device");
    const int M = 2 * (size_t)H * W * sizeof(float) <= prop0.sharedMemPerBlockOptin ? 16 : 32;
    std::vector<int> dealt;
    dealt.reserve(order.size());
    for (size_t lo = 0; lo < order.size();) {
      size_t hi = lo;
      while (hi < order.size() && sts[order[hi]].side == sts[order[lo]].side) ++hi;
      std::vector<std::vector<int>> bucket((size_t)M);
      for (size_t i = lo; i < hi; ++i) {
        const Stencil& st = sts[order[i]];
        const long long key = (long long)st.y0 * W + st.x0;
        bucket[(size_t)(((key % M) + M) % M)].push_back(order[i]);
      }
      for (size_t round = 0, left = hi - lo; left > 0; ++round)
        for (int r = 0; r < M; ++r)
          if (round < bucket[(size_t)r].size()) {
            dealt.push_back(bucket[(size_t)r][round]);
            --left;
          }
      lo = hi;
    }
    order.swap(dealt);
  }
  const int n_groups = (2 * U + 31) / 32;
  std::vector<int2> grp((size_t)n_groups);
  std::vector<int4> slot((size_t)n_groups * 32, make_int4(0, 0, -1, 0));
  int64_t taps = 0;
  for (int gi = 0; gi < n_groups; ++gi) {
    const int last = std::min(2 * U, (gi + 1) * 32) - 1;
    grp[gi] = make_int2((int)taps, sts[order[last]].side);   // sorted: the last lane has the widest patch
    taps += ((int64_t)grp[gi].y * grp[gi].y + TB - 1) / TB * TB;   // padded with zero weights
  }
  if (taps * 32 > (int64_t)INT32_MAX) return lgn_fail(nullptr, V1G_EINVAL, "v1g_lgn_create: stencil table too large");
  std::vector<float> w((size_t)taps * 32, 0.f);
  for (int i = 0; i < 2 * U; ++i) {
    const int gi = i >> 5, ln = i & 31, gside = grp[gi].y;
    const Stencil& st = sts[order[i]];
    slot[i] = make_int4(st.y0, st.x0, order[i], 0);
    // a narrower stencil sits in the top-left corner of the group's patch; the rest stays 0
    for (int dy = 0; dy < st.side; ++dy)
      for (int dx = 0; dx < st.side; ++dx)
        w[((size_t)grp[gi].x + (size_t)dy * gside + dx) * 32 + ln] = st.w[(size_t)dy * st.side + dx];
  }

  V1GLgn* l = new V1GLgn();
  l->n_units = U; l->height = H; l->width = W; l->len_dom = tb->len_dom; l->len_non_dom = tb->len_non_dom;
  cudaDeviceProp prop;
  if (cudaGetDevice(&l->device) != cudaSuccess || cudaGetDeviceProperties(&prop, l->device) != cudaSuccess) {
    delete l;
    return lgn_fail(nullptr, V1G_ECUDA, "v1g_lgn_create: no CUDA device");
  }
  l->n_sms = prop.multiProcessorCount;
  l->smem_optin = (int)prop.sharedMemPerBlockOptin;
  int rc = V1G_OK;
  l->n_groups = n_groups;
  if ((rc = lgn_upload(l, &l->st_grp, grp.data(), grp.size())) || (rc = lgn_upload(l, &l->st_slot, slot.data(), slot.size())) ||
      (rc = lgn_upload(l, &l->st_w, w.data(), w.size())) ||
      (rc = lgn_upload(l, &l->k_dom, tb->dom_temporal_kernels, (size_t)tb->len_dom * U)) ||
      (rc = lgn_upload(l, &l->k_non_dom, tb->non_dom_temporal_kernels, (size_t)tb->len_non_dom * U)) ||
      (rc = lgn_upload(l, &l->amp, tb->amplitude, (size_t)U)) ||
      (rc = lgn_upload(l, &l->non_dom_amp, tb->non_dom_amplitude, (size_t)U)) ||
      (rc = lgn_upload(l, &l->composite, tb->is_composite, (size_t)U)) ||
      (rc = lgn_upload(l, &l->spont, tb->spontaneous_firing_rates, (size_t)U))) {
    v1g_lgn_destroy(l);
    return rc;
  }
  *out = l;
  return V1G_OK;
}

extern "C" int v1g_lgn_destroy(V1GLgn* l) {
  if (!l) return V1G_OK;
  cudaFree(l->st_grp); cudaFree(l->st_slot); cudaFree(l->st_w); cudaFree(l->k_dom); cudaFree(l->k_non_dom);
  cudaFree(l->amp); cudaFree(l->non_dom_amp); cudaFree(l->composite); cudaFree(l->spont); cudaFree(l->spatial);
  delete l;
  return V1G_OK;
}

extern "C" int v1g_lgn_firing_rates(V1GLgn* l, const float* movie, int32_t n_frames, float* spatial_out,
                                    float* rates_out, void* stream) {
  if (!l || n_frames < 0) return lgn_fail(l, V1G_EINVAL, "v1g_lgn_firing_rates: bad argument");
  if (n_frames == 0) return V1G_OK;  // an empty movie: nothing to write, whatever the pointers
  if ((!spatial_out && !rates_out) || (!movie && !(spatial_out && rates_out)))
    return lgn_fail(l, V1G_EINVAL, "v1g_lgn_firing_rates: bad argument");
  cudaStream_t st = (cudaStream_t)stream;
  const int T = n_frames, U = l->n_units;
  float* spatial = spatial_out;
  if (!spatial) {
    const int64_t need = (int64_t)2 * T * U;
    if (need > l->spatial_cap) {
      cudaFree(l->spatial);
      l->spatial = nullptr;
      l->spatial_cap = 0;
      LGN_CUDA(l, cudaMalloc((void**)&l->spatial, (size_t)need * sizeof(float)));
      l->spatial_cap = need;
    }
    spatial = l->spatial;
  }
  const size_t frame_bytes = (size_t)l->height * l->width * sizeof(float);
  if (movie) {
    const int F = 2 * frame_bytes <= (size_t)l->smem_optin ? 2 : 1;
    const int in_smem = (size_t)F * frame_bytes <= (size_t)l->smem_optin ? 1 : 0;
    const size_t smem = in_smem ? F * frame_bytes : 0;
    auto kern = F == 2 ? lgn_spatial_kernel<2, true> : in_smem ? lgn_spatial_kernel<1, true> : lgn_spatial_kernel<1, false>;
    if (in_smem) LGN_CUDA(l, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int blocks = std::max(1, std::min((T + F - 1) / F, l->n_sms * (in_smem ? 1 : 4)));
    kern<<<blocks, 1024, smem, st>>>(movie, T, l->height, l->width, U, l->n_groups, l->st_grp, l->st_slot, l->st_w,
                                    spatial);
    v1g_count_launches(1);
  }
  if (rates_out) {
    dim3 grid((U + 255) / 256, (T + TT - 1) / TT);
    lgn_temporal_kernel<<<grid, 256, 0, st>>>(spatial, T, U, l->k_dom, l->len_dom, l->k_non_dom, l->len_non_dom, l->amp,
                                              l->non_dom_amp, l->composite, l->spont, rates_out);
    v1g_count_launches(1);
  }
  LGN_CUDA(l, cudaGetLastError());
  return V1G_OK;
}

extern "C" const char* v1g_lgn_last_error(const V1GLgn* l) { return l ? l->err.c_str() : v1g_last_error(nullptr); }
