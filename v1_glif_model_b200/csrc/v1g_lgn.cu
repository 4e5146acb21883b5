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
// with taps outside the frame dropped (they are the zero padding).  A thread block takes one frame
// into shared memory (a 120 x 240 frame is 115 KB) and evaluates every stencil from there, so the
// movie is read from HBM once.  The temporal filter keeps a sliding window per thread: TT outputs of
// one unit per thread reuse every loaded sample and kernel value TT times.
#include <math.h>

#include <vector>

#include "v1g_internal.h"

struct V1GLgn {
  int n_units = 0, height = 0, width = 0, len_dom = 0, len_non_dom = 0;
  int device = 0, n_sms = 0, smem_optin = 0;
  // stencils of the dominant [0, U) and non-dominant [U, 2U) subfields
  int32_t* st_off = nullptr;   // [2U + 1] first weight of each stencil
  int32_t* st_geo = nullptr;   // [2U][3] = (y0, x0, side)
  float* st_w = nullptr;       // weights, row-major side x side
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

// one block per frame: the frame goes to shared memory, every (unit, subfield) stencil is evaluated
// from it; out[s][t][u]
__global__ void __launch_bounds__(512) lgn_spatial_kernel(const float* __restrict__ movie, int T, int H, int W, int U,
                                                          const int32_t* __restrict__ st_off,
                                                          const int32_t* __restrict__ st_geo,
                                                          const float* __restrict__ st_w, float* __restrict__ out,
                                                          int frame_in_smem) {
  extern __shared__ float frame_s[];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const float* frame = movie + (int64_t)t * H * W;
    if (frame_in_smem) {
      __syncthreads();
      for (int i = threadIdx.x; i < H * W; i += blockDim.x) frame_s[i] = frame[i];
      __syncthreads();
      frame = frame_s;
    }
    for (int su = threadIdx.x; su < 2 * U; su += blockDim.x) {
      const int y0 = st_geo[3 * su], x0 = st_geo[3 * su + 1], side = st_geo[3 * su + 2];
      const float* w = st_w + st_off[su];
      float acc = 0.f;
      for (int dy = 0; dy < side; ++dy) {
        const int y = y0 + dy;
        if (y < 0 || y >= H) continue;
        const float* row = frame + y * W;
        for (int dx = 0; dx < side; ++dx) {
          const int x = x0 + dx;
          if (x >= 0 && x < W) acc += w[dy * side + dx] * row[x];
        }
      }
      const int s = su >= U ? 1 : 0, u = su - s * U;
      out[((int64_t)s * T + t) * U + u] = acc;
    }
  }
}

// rates[t][u] = relu(amp * f_dom + spont) + composite * relu(nd_amp * f_nd + spont), f = causal filter
// of the unit's samples: f[t] = sum_j K[j] * s[t - (L - 1) + j] with s = 0 before the movie starts
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
  for (int i = 0; i < TT; ++i) f[0][i] = f[1][i] = 0.f;
  for (int s = 0; s < 2; ++s) {
    const float* kern = s ? k_nd : k_dom;
    const int L = s ? len_nd : len_dom;
    const float* smp = spatial + (int64_t)s * T * U;
    // sample index q runs over t0 - (L - 1) .. t0 + TT - 1; output i uses kernel tap j = q - (t0 + i) + L - 1
    for (int q = t0 - (L - 1); q < t0 + TT; ++q) {
      if (q < 0 || q >= T) continue;
      const float v = smp[(int64_t)q * U + u];
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        const int j = q - (t0 + i) + L - 1;
        if (j >= 0 && j < L) f[s][i] += kern[(int64_t)j * U + u] * v;
      }
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
  std::vector<int32_t> off((size_t)2 * U + 1, 0), geo((size_t)2 * U * 3);
  std::vector<float> w;
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
    off[su] = (int32_t)w.size();
    geo[3 * su] = yf - r;
    geo[3 * su + 1] = xf - r;
    geo[3 * su + 2] = side;
    for (double v : e) w.push_back((float)v);
  }
  off[(size_t)2 * U] = (int32_t)w.size();

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
  if ((rc = lgn_upload(l, &l->st_off, off.data(), off.size())) || (rc = lgn_upload(l, &l->st_geo, geo.data(), geo.size())) ||
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
  cudaFree(l->st_off); cudaFree(l->st_geo); cudaFree(l->st_w); cudaFree(l->k_dom); cudaFree(l->k_non_dom);
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
  const int in_smem = frame_bytes <= (size_t)l->smem_optin ? 1 : 0;
  if (in_smem)
    LGN_CUDA(l, cudaFuncSetAttribute(lgn_spatial_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)frame_bytes));
  if (movie) {
    lgn_spatial_kernel<<<std::min(T, l->n_sms * 4), 512, in_smem ? frame_bytes : 0, st>>>(
        movie, T, l->height, l->width, U, l->st_off, l->st_geo, l->st_w, spatial, in_smem);
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
