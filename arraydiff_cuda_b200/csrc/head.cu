// Classifier head after the spatial stages: average pooling (global or windowed) and the fully connected
// layer.  Small, HBM- / latency-bound kernels: the head works on [batch][channels] vectors.
//   average pool:  CudnnPool2DOp with kAveragePool (reference src/op.cc:3346-3633; zoo.cc:1843-1852)
//   linear:        CublasLinearOp (reference src/op.cc:1199-1340: cublasSgemm + bias add)
#include "common.cuh"

namespace adk {

struct HView { char* base; long long sn, sc, sy, sx; };
static HView hview(const ad_tensor4* t) { return HView{(char*)t->base, t->sn, t->sc, t->sy, t->sx}; }

struct AvgP {
  HView x, y;
  uint32_t N, C, H, W, P, Q, kh, kw, sh, sw;
  int c_fastest, accumulate;
};

// one thread per output element; the window mean is accumulated in row-major order
template <typename T>
__global__ void __launch_bounds__(256) avgpool_fwd_kernel(AvgP p) {
  const uint32_t total = p.N * p.C * p.P * p.Q, nt = gridDim.x * blockDim.x;
  const float inv = 1.0f / (float)(p.kh * p.kw);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, q, s, r = i;
    if (p.c_fastest) { c = r % p.C; r /= p.C; s = r % p.Q; r /= p.Q; q = r % p.P; n = r / p.P; }
    else { s = r % p.Q; r /= p.Q; q = r % p.P; r /= p.P; c = r % p.C; n = r / p.C; }
    const T* X = (const T*)p.x.base + n * p.x.sn + c * p.x.sc;
    float acc = 0.f;
    for (uint32_t a = 0; a < p.kh; ++a)
      for (uint32_t b = 0; b < p.kw; ++b) acc += ld_f(X + (q * p.sh + a) * p.x.sy + (s * p.sw + b) * p.x.sx);
    st_f((T*)p.y.base + n * p.y.sn + c * p.y.sc + q * p.y.sy + s * p.y.sx, acc * inv);
  }
}
// one thread per input element gathers from the windows over it
template <typename T>
__global__ void __launch_bounds__(256) avgpool_bwd_kernel(AvgP p) {
  const uint32_t total = p.N * p.C * p.H * p.W, nt = gridDim.x * blockDim.x;
  const float inv = 1.0f / (float)(p.kh * p.kw);
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, y, x, r = i;
    if (p.c_fastest) { c = r % p.C; r /= p.C; x = r % p.W; r /= p.W; y = r % p.H; n = r / p.H; }
    else { x = r % p.W; r /= p.W; y = r % p.H; r /= p.H; c = r % p.C; n = r / p.C; }
    const uint32_t q_lo = y + 1 > p.kh ? (y + 1 - p.kh + p.sh - 1) / p.sh : 0;
    const uint32_t s_lo = x + 1 > p.kw ? (x + 1 - p.kw + p.sw - 1) / p.sw : 0;
    const T* G = (const T*)p.y.base + n * p.y.sn + c * p.y.sc;
    float acc = 0.f;
    for (uint32_t q = q_lo; q < p.P && q * p.sh <= y; ++q)
      for (uint32_t s = s_lo; s < p.Q && s * p.sw <= x; ++s) acc += ld_f(G + q * p.y.sy + s * p.y.sx);
    acc *= inv;
    T* o = (T*)p.x.base + n * p.x.sn + c * p.x.sc + y * p.x.sy + x * p.x.sx;
    st_f(o, p.accumulate ? ld_f(o) + acc : acc);
  }
}

static int avg_params(const ad_tensor4* x, const ad_tensor4* y, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, AvgP& p) {
  if (!x || !y || !x->base || !y->base || kh == 0 || kw == 0 || sh == 0 || sw == 0) return AD_ERR_BAD_ARG;
  if (x->H < kh || x->W < kw) return AD_ERR_BAD_ARG;
  const uint32_t P = (x->H - kh) / sh + 1, Q = (x->W - kw) / sw + 1;
  if (y->N != x->N || y->C != x->C || y->H != P || y->W != Q || y->dtype != x->dtype) return AD_ERR_BAD_ARG;
  if ((size_t)x->N * x->C * x->H * x->W >= (1ull << 32)) return AD_ERR_LIMIT;
  p.x = hview(x); p.y = hview(y);
  p.N = x->N; p.C = x->C; p.H = x->H; p.W = x->W; p.P = P; p.Q = Q; p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw;
  return AD_OK;
}

// ------------------------------------------------------------------ fully connected
// y[b][o] = bias[o] + sum_i x[b][i] * w[o][i]: one warp per output, lanes stride over i, shuffle sum.
template <typename T>
__global__ void __launch_bounds__(256) linear_fwd_kernel(uint32_t B, uint32_t I, uint32_t O, const T* __restrict__ x,
                                                         const float* __restrict__ w, const float* __restrict__ bias, T* y) {
  const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31, nw = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t j = warp; j < B * O; j += nw) {
    const uint32_t b = j / O, o = j - b * O;
    float acc = 0.f;
    for (uint32_t i = lane; i < I; i += 32) acc = fmaf(ld_f(x + (size_t)b * I + i), w[(size_t)o * I + i], acc);
    acc = warp_sum(acc);
    if (lane == 0) st_f(y + (size_t)b * O + o, acc + (bias ? bias[o] : 0.f));
  }
}
// dx[b][i] (+)= sum_o dy[b][o] * w[o][i]: one thread per (b, i), coalesced over i
template <typename T>
__global__ void __launch_bounds__(256) linear_dx_kernel(uint32_t B, uint32_t I, uint32_t O, const T* __restrict__ dy,
                                                        const float* __restrict__ w, T* dx, int accumulate) {
  const uint32_t total = B * I, nt = gridDim.x * blockDim.x;
  for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < total; j += nt) {
    const uint32_t b = j / I, i = j - b * I;
    float acc = 0.f;
    for (uint32_t o = 0; o < O; ++o) acc = fmaf(ld_f(dy + (size_t)b * O + o), w[(size_t)o * I + i], acc);
    st_f(dx + j, accumulate ? ld_f(dx + j) + acc : acc);
  }
}
// dw[o][i] (+)= sum_b dy[b][o] * x[b][i]; db[o] (+)= sum_b dy[b][o]: one thread per (o, i), batch in order
template <typename T>
__global__ void __launch_bounds__(256) linear_dw_kernel(uint32_t B, uint32_t I, uint32_t O, const T* __restrict__ x,
                                                        const T* __restrict__ dy, float* dw, float* db, int accumulate) {
  const uint32_t total = O * I, nt = gridDim.x * blockDim.x;
  for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < total; j += nt) {
    const uint32_t o = j / I, i = j - o * I;
    float acc = 0.f, accb = 0.f;
    for (uint32_t b = 0; b < B; ++b) {
      const float g = ld_f(dy + (size_t)b * O + o);
      acc = fmaf(g, ld_f(x + (size_t)b * I + i), acc);
      accb += g;
    }
    dw[j] = accumulate ? dw[j] + acc : acc;
    if (db && i == 0) db[o] = accumulate ? db[o] + accb : accb;
  }
}

}  // namespace adk

using namespace adk;

extern "C" int ad_avgpool2d_fwd(const ad_tensor4* x, const ad_tensor4* y, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw,
                                void* stream) {
  AvgP p{};
  int st = avg_params(x, y, kh, kw, sh, sw, p);
  if (st != AD_OK) return st;
  const size_t total = (size_t)p.N * p.C * p.P * p.Q;
  if (total == 0) return AD_OK;
  p.c_fastest = y->sc == 1 && y->C > 1;
  AD_DISPATCH_DTYPE(x->dtype, (avgpool_fwd_kernel<T><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  count_launch();
  return launch_status();
}

extern "C" int ad_avgpool2d_bwd(const ad_tensor4* dy, const ad_tensor4* dx, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw,
                                int32_t accumulate, void* stream) {
  AvgP p{};
  int st = avg_params(dx, dy, kh, kw, sh, sw, p);
  if (st != AD_OK) return st;
  const size_t total = (size_t)p.N * p.C * p.H * p.W;
  if (total == 0) return AD_OK;
  p.c_fastest = dx->sc == 1 && dx->C > 1;
  p.accumulate = accumulate;
  AD_DISPATCH_DTYPE(dx->dtype, (avgpool_bwd_kernel<T><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  count_launch();
  return launch_status();
}

extern "C" int ad_linear_fwd(int32_t dtype, uint32_t batch, uint32_t in_features, uint32_t out_features, const void* x,
                             const float* w, const float* bias, void* y, void* stream) {
  if (!x || !w || !y) return AD_ERR_BAD_ARG;
  if ((size_t)batch * out_features >= (1ull << 31) || (size_t)batch * in_features >= (1ull << 31)) return AD_ERR_LIMIT;
  if (batch == 0 || out_features == 0) return AD_OK;
  const size_t warps = (size_t)batch * out_features;
  AD_DISPATCH_DTYPE(dtype, (linear_fwd_kernel<T><<<grid_for(warps * 32, 256, 16), 256, 0, as_stream(stream)>>>(
                               batch, in_features, out_features, (const T*)x, w, bias, (T*)y)));
  count_launch();
  return launch_status();
}

extern "C" int ad_linear_bwd(int32_t dtype, uint32_t batch, uint32_t in_features, uint32_t out_features, const void* x,
                             const float* w, const void* dy, void* dx, float* dw, float* db, int32_t accumulate_dx,
                             int32_t accumulate_dw, void* stream) {
  if (!x || !w || !dy) return AD_ERR_BAD_ARG;
  if ((size_t)batch * out_features >= (1ull << 31) || (size_t)batch * in_features >= (1ull << 31) ||
      (size_t)in_features * out_features >= (1ull << 31))
    return AD_ERR_LIMIT;
  if (batch == 0) return AD_OK;
  cudaStream_t s = as_stream(stream);
  if (dx) {
    AD_DISPATCH_DTYPE(dtype, (linear_dx_kernel<T><<<grid_for((size_t)batch * in_features, 256, 16), 256, 0, s>>>(
                                 batch, in_features, out_features, (const T*)dy, w, (T*)dx, accumulate_dx)));
    count_launch();
  }
  if (dw) {
    AD_DISPATCH_DTYPE(dtype, (linear_dw_kernel<T><<<grid_for((size_t)in_features * out_features, 256, 16), 256, 0, s>>>(
                                 batch, in_features, out_features, (const T*)x, (const T*)dy, dw, db, accumulate_dw)));
    count_launch();
  }
  return launch_status();
}
