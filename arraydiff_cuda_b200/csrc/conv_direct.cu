// fp32 NCHW convolution with fp32 FMA accumulate: the exact-precision path (max-relative
// 1e-5 against a double-accumulating CPU result) used where the graph boundary is fp32 and
// for cross-checking the tensor-core path.  Not the throughput path: that is conv_tc.cu.
#include "common.cuh"

namespace adk {

struct ConvG {
  uint32_t N, C, H, W, K, kh, kw, sh, sw, dh, dw, ph, pw, P, Q;
  long long y_pitch, y_plane;
  int relu, accumulate;
};

__global__ void __launch_bounds__(256) conv_fprop_f32(ConvG g, const float* __restrict__ x, const float* __restrict__ w,
                                                      const float* __restrict__ bias, float* y) {
  const size_t total = (size_t)g.N * g.K * g.P * g.Q, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += nt) {
    uint32_t s = (uint32_t)(idx % g.Q);
    size_t r = idx / g.Q;
    uint32_t q = (uint32_t)(r % g.P); r /= g.P;
    uint32_t k = (uint32_t)(r % g.K), n = (uint32_t)(r / g.K);
    float acc = bias ? bias[k] : 0.f;
    for (uint32_t c = 0; c < g.C; ++c) {
      float part = 0.f;  // per-channel partial keeps the running sum short
      const float* xp = x + ((size_t)n * g.C + c) * g.H * g.W;
      const float* wp = w + ((size_t)k * g.C + c) * g.kh * g.kw;
      for (uint32_t i = 0; i < g.kh; ++i) {
        int yy = (int)(q * g.sh + i * g.dh) - (int)g.ph;
        if (yy < 0 || yy >= (int)g.H) continue;
        for (uint32_t j = 0; j < g.kw; ++j) {
          int xx = (int)(s * g.sw + j * g.dw) - (int)g.pw;
          if (xx < 0 || xx >= (int)g.W) continue;
          part = fmaf(xp[(size_t)yy * g.W + xx], wp[i * g.kw + j], part);
        }
      }
      acc += part;
    }
    if (g.relu) acc = fmaxf(acc, 0.f);
    y[((size_t)n * g.K + k) * g.y_plane + (size_t)q * g.y_pitch + s] = acc;
  }
}

__global__ void __launch_bounds__(256) conv_dgrad_f32(ConvG g, const float* __restrict__ dy, const float* __restrict__ w,
                                                      float* dx) {
  const size_t total = (size_t)g.N * g.C * g.H * g.W, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += nt) {
    uint32_t xx = (uint32_t)(idx % g.W);
    size_t r = idx / g.W;
    uint32_t yy = (uint32_t)(r % g.H); r /= g.H;
    uint32_t c = (uint32_t)(r % g.C), n = (uint32_t)(r / g.C);
    float acc = 0.f;
    for (uint32_t i = 0; i < g.kh; ++i) {
      int t = (int)(yy + g.ph) - (int)(i * g.dh);
      if (t < 0 || t % (int)g.sh) continue;
      uint32_t q = (uint32_t)t / g.sh;
      if (q >= g.P) continue;
      for (uint32_t j = 0; j < g.kw; ++j) {
        int u = (int)(xx + g.pw) - (int)(j * g.dw);
        if (u < 0 || u % (int)g.sw) continue;
        uint32_t s = (uint32_t)u / g.sw;
        if (s >= g.Q) continue;
        float part = 0.f;
        for (uint32_t k = 0; k < g.K; ++k)
          part = fmaf(dy[((size_t)n * g.K + k) * g.y_plane + (size_t)q * g.y_pitch + s],
                      w[(((size_t)k * g.C + c) * g.kh + i) * g.kw + j], part);
        acc += part;
      }
    }
    if (g.accumulate) acc += dx[idx];
    dx[idx] = acc;
  }
}

// One block per (k, c): every thread sums a strided share of the (n, q, s) positions for all
// kh*kw taps (at most 49 here), then a fixed-order tree reduction.
template <int MAXT>
__global__ void __launch_bounds__(256) conv_wgrad_f32(ConvG g, const float* __restrict__ x, const float* __restrict__ dy,
                                                      float* dw) {
  const uint32_t k = blockIdx.x / g.C, c = blockIdx.x % g.C;
  const uint32_t taps = g.kh * g.kw;
  float acc[MAXT];
#pragma unroll
  for (int t = 0; t < MAXT; ++t) acc[t] = 0.f;
  const size_t per = (size_t)g.N * g.P * g.Q;
  for (size_t idx = threadIdx.x; idx < per; idx += blockDim.x) {
    uint32_t s = (uint32_t)(idx % g.Q);
    size_t r = idx / g.Q;
    uint32_t q = (uint32_t)(r % g.P), n = (uint32_t)(r / g.P);
    const float d = dy[((size_t)n * g.K + k) * g.y_plane + (size_t)q * g.y_pitch + s];
    const float* xp = x + ((size_t)n * g.C + c) * g.H * g.W;
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
      if (t < (int)taps) {
        uint32_t i = t / g.kw, j = t % g.kw;
        int yy = (int)(q * g.sh + i * g.dh) - (int)g.ph, xx = (int)(s * g.sw + j * g.dw) - (int)g.pw;
        if (yy >= 0 && yy < (int)g.H && xx >= 0 && xx < (int)g.W) acc[t] = fmaf(d, xp[(size_t)yy * g.W + xx], acc[t]);
      }
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int t = 0; t < MAXT; ++t) {
    if (t < (int)taps) {
      float v = warp_sum(acc[t]);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
      __syncthreads();
      if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int wv = 0; wv < 8; ++wv) tot += red[wv];
        float* o = dw + ((size_t)k * g.C + c) * taps + t;
        *o = g.accumulate ? *o + tot : tot;
      }
      __syncthreads();
    }
  }
}

__global__ void __launch_bounds__(256) conv_bgrad_f32(ConvG g, const float* __restrict__ dy, float* db) {
  const uint32_t k = blockIdx.x;
  float acc = 0.f;
  const size_t per = (size_t)g.N * g.P * g.Q;
  for (size_t idx = threadIdx.x; idx < per; idx += blockDim.x) {
    uint32_t s = (uint32_t)(idx % g.Q);
    size_t r = idx / g.Q;
    uint32_t q = (uint32_t)(r % g.P), n = (uint32_t)(r / g.P);
    acc += dy[((size_t)n * g.K + k) * g.y_plane + (size_t)q * g.y_pitch + s];
  }
  __shared__ float red[8];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int wv = 0; wv < 8; ++wv) tot += red[wv];
    db[k] = g.accumulate ? db[k] + tot : tot;
  }
}

static int geometry(const ad_conv2d_args* a, ConvG& g) {
  if (!a) return AD_ERR_BAD_ARG;
  if (a->N == 0 || a->C == 0 || a->H == 0 || a->W == 0 || a->K == 0 || a->kh == 0 || a->kw == 0) return AD_ERR_BAD_ARG;
  if (a->stride_h == 0 || a->stride_w == 0 || a->dil_h == 0 || a->dil_w == 0) return AD_ERR_BAD_ARG;
  const long long eh = (long long)a->H + 2ll * a->pad_h - (long long)a->dil_h * (a->kh - 1) - 1;
  const long long ew = (long long)a->W + 2ll * a->pad_w - (long long)a->dil_w * (a->kw - 1) - 1;
  if (eh < 0 || ew < 0) return AD_ERR_BAD_ARG;
  g = ConvG{a->N, a->C, a->H, a->W, a->K, a->kh, a->kw, a->stride_h, a->stride_w, a->dil_h, a->dil_w, a->pad_h, a->pad_w,
            (uint32_t)(eh / a->stride_h + 1), (uint32_t)(ew / a->stride_w + 1), 0, 0, a->relu, a->accumulate};
  g.y_pitch = a->y_pitch ? a->y_pitch : g.Q;
  g.y_plane = a->y_plane ? a->y_plane : (long long)g.P * g.Q;
  return AD_OK;
}

int conv_direct_fprop(const ad_conv2d_args* a, cudaStream_t s) {
  ConvG g;
  int st = geometry(a, g);
  if (st != AD_OK) return st;
  if (!a->x || !a->w || !a->y) return AD_ERR_BAD_ARG;
  if (a->out_row_count) return AD_ERR_UNSUPPORTED;   // row ranges: tensor-core path only
  const size_t total = (size_t)g.N * g.K * g.P * g.Q;
  conv_fprop_f32<<<grid_for(total, 256, 16), 256, 0, s>>>(g, (const float*)a->x, (const float*)a->w, a->bias, (float*)a->y);
  count_launch();
  return launch_status();
}

int conv_direct_dgrad(const ad_conv2d_args* a, cudaStream_t s) {
  ConvG g;
  int st = geometry(a, g);
  if (st != AD_OK) return st;
  if (!a->y || !a->w || !a->dx) return AD_ERR_BAD_ARG;
  if (a->dx_col_count) return AD_ERR_UNSUPPORTED;   // column ranges: tensor-core path only
  const size_t total = (size_t)g.N * g.C * g.H * g.W;
  conv_dgrad_f32<<<grid_for(total, 256, 16), 256, 0, s>>>(g, (const float*)a->y, (const float*)a->w, (float*)a->dx);
  count_launch();
  return launch_status();
}

int conv_direct_wgrad(const ad_conv2d_args* a, cudaStream_t s) {
  ConvG g;
  int st = geometry(a, g);
  if (st != AD_OK) return st;
  if (!a->x || !a->y || !a->dw) return AD_ERR_BAD_ARG;
  const uint32_t taps = g.kh * g.kw;
  if (taps <= 9) conv_wgrad_f32<9><<<g.K * g.C, 256, 0, s>>>(g, (const float*)a->x, (const float*)a->y, (float*)a->dw);
  else if (taps <= 49) conv_wgrad_f32<49><<<g.K * g.C, 256, 0, s>>>(g, (const float*)a->x, (const float*)a->y, (float*)a->dw);
  else return AD_ERR_UNSUPPORTED;
  count_launch();
  if (a->db) {
    conv_bgrad_f32<<<g.K, 256, 0, s>>>(g, (const float*)a->y, a->db);
    count_launch();
  }
  return launch_status();
}

}  // namespace adk
