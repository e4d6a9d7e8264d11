// Bilinear x`scale` upsample (half-pixel centres, edges clamped) of a strip of a 4-D tensor and its
// gradient, on strided views.  The reference has no such operator; it is the segmentation head of the
// 1024x2048 configuration (logits at 1/8 resolution -> full resolution before the per-pixel loss).
//
// Strip form: the views hold rows [x_row0, x_row0 + x.H) of an input whose full height is in_rows_total
// and rows [y_row0, y_row0 + y.H) of the upsampled output; source rows are computed in global
// coordinates, so a strip with one halo row on each inner edge gives exactly the rows of the
// unpartitioned result.  HBM-bound: the output is scale^2 times the input.
#include "common.cuh"

namespace adk {

struct UpView { char* base; long long sn, sc, sy, sx; };
static UpView upview(const ad_tensor4* t) { return UpView{(char*)t->base, t->sn, t->sc, t->sy, t->sx}; }

struct UpP {
  UpView x, y;            // x: low-resolution side, y: high-resolution side
  uint32_t N, C, XH, XW, YH, YW, scale;
  int32_t x_row0;
  uint32_t in_rows_total, y_row0;
  int c_fastest, accumulate;
};

// source cell pair and weight for output index o (global), as torch's align_corners = false
__device__ __forceinline__ void bilin_src(uint32_t o, float inv_scale, uint32_t in_size, int& i0, int& i1, float& f) {
  float src = ((float)o + 0.5f) * inv_scale - 0.5f;
  if (src < 0.f) src = 0.f;
  int a = (int)floorf(src);
  if (a > (int)in_size - 1) a = (int)in_size - 1;
  i0 = a;
  i1 = a + 1 < (int)in_size ? a + 1 : (int)in_size - 1;
  f = src - (float)a;
}

template <typename T>
__global__ void __launch_bounds__(256) upsample_fwd_kernel(UpP p) {
  const uint32_t total = p.N * p.C * p.YH * p.YW, nt = gridDim.x * blockDim.x;
  const float inv = 1.0f / (float)p.scale;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, oy, ox, r = i;
    if (p.c_fastest) { c = r % p.C; r /= p.C; ox = r % p.YW; r /= p.YW; oy = r % p.YH; n = r / p.YH; }
    else { ox = r % p.YW; r /= p.YW; oy = r % p.YH; r /= p.YH; c = r % p.C; n = r / p.C; }
    int y0, y1, x0, x1;
    float fy, fx;
    bilin_src(p.y_row0 + oy, inv, p.in_rows_total, y0, y1, fy);
    bilin_src(ox, inv, p.XW, x0, x1, fx);
    y0 -= p.x_row0; y1 -= p.x_row0;
    const T* X = (const T*)p.x.base + n * p.x.sn + c * p.x.sc;
    const float a = ld_f(X + y0 * p.x.sy + x0 * p.x.sx), b = ld_f(X + y0 * p.x.sy + x1 * p.x.sx);
    const float d = ld_f(X + y1 * p.x.sy + x0 * p.x.sx), e = ld_f(X + y1 * p.x.sy + x1 * p.x.sx);
    const float v = (1.f - fy) * ((1.f - fx) * a + fx * b) + fy * ((1.f - fx) * d + fx * e);
    st_f((T*)p.y.base + n * p.y.sn + c * p.y.sc + oy * p.y.sy + ox * p.y.sx, v);
  }
}

// Gather form of the gradient: one thread per low-resolution element sums, in a fixed order, the
// high-resolution gradients whose source pair contains it -- no atomics, reproducible.
template <typename T>
__global__ void __launch_bounds__(256) upsample_bwd_kernel(UpP p) {
  const uint32_t total = p.N * p.C * p.XH * p.XW, nt = gridDim.x * blockDim.x;
  const float inv = 1.0f / (float)p.scale;
  const int s = (int)p.scale;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, yl, xl, r = i;
    if (p.c_fastest) { c = r % p.C; r /= p.C; xl = r % p.XW; r /= p.XW; yl = r % p.XH; n = r / p.XH; }
    else { xl = r % p.XW; r /= p.XW; yl = r % p.XH; r /= p.XH; c = r % p.C; n = r / p.C; }
    const int yg = (int)yl + p.x_row0, xg = (int)xl;
    float acc = 0.f;
    if (yg >= 0 && yg < (int)p.in_rows_total) {
      // candidates: outputs whose source coordinate lies in (g - 1, g + 1); edge cells also take the clamped ones
      int oy_lo = yg == 0 ? 0 : (yg - 1) * s, oy_hi = yg == (int)p.in_rows_total - 1 ? (int)p.in_rows_total * s - 1 : (yg + 2) * s - 1;
      int ox_lo = xg == 0 ? 0 : (xg - 1) * s, ox_hi = xg == (int)p.XW - 1 ? (int)p.XW * s - 1 : (xg + 2) * s - 1;
      if (oy_lo < (int)p.y_row0) oy_lo = (int)p.y_row0;
      if (oy_hi > (int)(p.y_row0 + p.YH) - 1) oy_hi = (int)(p.y_row0 + p.YH) - 1;
      const T* G = (const T*)p.y.base + n * p.y.sn + c * p.y.sc;
      for (int oy = oy_lo; oy <= oy_hi; ++oy) {
        int y0, y1;
        float fy;
        bilin_src((uint32_t)oy, inv, p.in_rows_total, y0, y1, fy);
        const float wy = (y0 == yg ? 1.f - fy : 0.f) + (y1 == yg ? fy : 0.f);
        if (wy == 0.f) continue;
        float row = 0.f;
        for (int ox = ox_lo; ox <= ox_hi; ++ox) {
          int x0, x1;
          float fx;
          bilin_src((uint32_t)ox, inv, p.XW, x0, x1, fx);
          const float wx = (x0 == xg ? 1.f - fx : 0.f) + (x1 == xg ? fx : 0.f);
          if (wx != 0.f) row = fmaf(wx, ld_f(G + (oy - (int)p.y_row0) * p.y.sy + ox * p.y.sx), row);
        }
        acc = fmaf(wy, row, acc);
      }
    }
    T* o = (T*)p.x.base + n * p.x.sn + c * p.x.sc + yl * p.x.sy + xl * p.x.sx;
    st_f(o, p.accumulate ? ld_f(o) + acc : acc);
  }
}

// Channel-fastest views: one thread per PIXEL computes the source cells and weights once and walks the channels
// (adjacent threads own adjacent pixels, so a warp's accesses cover runs of whole pixels).
template <typename T>
__global__ void __launch_bounds__(256) upsample_fwd_px_kernel(UpP p) {
  const uint32_t total = p.N * p.YH * p.YW, nt = gridDim.x * blockDim.x;
  const float inv = 1.0f / (float)p.scale;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t ox = i % p.YW, r = i / p.YW, oy = r % p.YH, n = r / p.YH;
    int y0, y1, x0, x1;
    float fy, fx;
    bilin_src(p.y_row0 + oy, inv, p.in_rows_total, y0, y1, fy);
    bilin_src(ox, inv, p.XW, x0, x1, fx);
    y0 -= p.x_row0; y1 -= p.x_row0;
    const T* X = (const T*)p.x.base + n * p.x.sn;
    const T *pa = X + y0 * p.x.sy + x0 * p.x.sx, *pb = X + y0 * p.x.sy + x1 * p.x.sx;
    const T *pd = X + y1 * p.x.sy + x0 * p.x.sx, *pe = X + y1 * p.x.sy + x1 * p.x.sx;
    T* o = (T*)p.y.base + n * p.y.sn + oy * p.y.sy + ox * p.y.sx;
    for (uint32_t c = 0; c < p.C; ++c) {
      const float v = (1.f - fy) * ((1.f - fx) * ld_f(pa + c) + fx * ld_f(pb + c)) + fy * ((1.f - fx) * ld_f(pd + c) + fx * ld_f(pe + c));
      st_f(o + c, v);
    }
  }
}
// Gradient, channel-fastest: one thread per low-resolution pixel and group of up to 8 channels; the weights
// of a candidate are computed once for the group.  Same candidates and order as the element form.
template <typename T>
__global__ void __launch_bounds__(256) upsample_bwd_px_kernel(UpP p) {
  const uint32_t G = (p.C + 7) / 8, total = p.N * p.XH * p.XW * G, nt = gridDim.x * blockDim.x;
  const float inv = 1.0f / (float)p.scale;
  const int s = (int)p.scale;
  for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t cg = i % G;
    uint32_t r = i / G;
    const uint32_t xl = r % p.XW; r /= p.XW;
    const uint32_t yl = r % p.XH, n = r / p.XH;
    const uint32_t c0 = cg * 8, nc = p.C - c0 < 8 ? p.C - c0 : 8;
    const int yg = (int)yl + p.x_row0, xg = (int)xl;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (yg >= 0 && yg < (int)p.in_rows_total) {
      int oy_lo = yg == 0 ? 0 : (yg - 1) * s, oy_hi = yg == (int)p.in_rows_total - 1 ? (int)p.in_rows_total * s - 1 : (yg + 2) * s - 1;
      int ox_lo = xg == 0 ? 0 : (xg - 1) * s, ox_hi = xg == (int)p.XW - 1 ? (int)p.XW * s - 1 : (xg + 2) * s - 1;
      if (oy_lo < (int)p.y_row0) oy_lo = (int)p.y_row0;
      if (oy_hi > (int)(p.y_row0 + p.YH) - 1) oy_hi = (int)(p.y_row0 + p.YH) - 1;
      const T* Gp = (const T*)p.y.base + n * p.y.sn + c0;
      for (int oy = oy_lo; oy <= oy_hi; ++oy) {
        int y0, y1;
        float fy;
        bilin_src((uint32_t)oy, inv, p.in_rows_total, y0, y1, fy);
        const float wy = (y0 == yg ? 1.f - fy : 0.f) + (y1 == yg ? fy : 0.f);
        if (wy == 0.f) continue;
        float row[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) row[j] = 0.f;
        for (int ox = ox_lo; ox <= ox_hi; ++ox) {
          int x0, x1;
          float fx;
          bilin_src((uint32_t)ox, inv, p.XW, x0, x1, fx);
          const float wx = (x0 == xg ? 1.f - fx : 0.f) + (x1 == xg ? fx : 0.f);
          if (wx == 0.f) continue;
          const T* gp = Gp + (oy - (int)p.y_row0) * p.y.sy + ox * p.y.sx;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if ((uint32_t)j < nc) row[j] = fmaf(wx, ld_f(gp + j), row[j]);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = fmaf(wy, row[j], acc[j]);
      }
    }
    T* o = (T*)p.x.base + n * p.x.sn + yl * p.x.sy + xl * p.x.sx + c0;
    for (uint32_t j = 0; j < nc; ++j) st_f(o + j, p.accumulate ? ld_f(o + j) + acc[j] : acc[j]);
  }
}

static int up_params(const ad_tensor4* lo, const ad_tensor4* hi, uint32_t scale, int32_t x_row0, uint32_t in_rows_total,
                     uint32_t y_row0, UpP& p) {
  if (!lo || !hi || !lo->base || !hi->base || scale == 0 || in_rows_total == 0) return AD_ERR_BAD_ARG;
  if (lo->N != hi->N || lo->C != hi->C || lo->dtype != hi->dtype || hi->W != lo->W * scale) return AD_ERR_BAD_ARG;
  if ((size_t)hi->N * hi->C * hi->H * hi->W >= (1ull << 32) || (size_t)in_rows_total * scale >= (1ull << 31)) return AD_ERR_LIMIT;
  if ((size_t)y_row0 + hi->H > (size_t)in_rows_total * scale) return AD_ERR_BAD_ARG;
  // every source row the high-resolution rows refer to must lie inside the low-resolution view
  if (hi->H > 0) {
    auto src_rows = [&](uint32_t o, long long& a, long long& b) {
      double src = ((double)o + 0.5) / (double)scale - 0.5;
      if (src < 0.0) src = 0.0;
      long long i0 = (long long)src;
      if (i0 > (long long)in_rows_total - 1) i0 = (long long)in_rows_total - 1;
      a = i0;
      b = i0 + 1 < (long long)in_rows_total ? i0 + 1 : (long long)in_rows_total - 1;
    };
    long long a0, b0, a1, b1;
    src_rows(y_row0, a0, b0);
    src_rows(y_row0 + hi->H - 1, a1, b1);
    if (a0 < x_row0 || b1 >= (long long)x_row0 + lo->H) return AD_ERR_BAD_ARG;
  }
  p.x = upview(lo); p.y = upview(hi);
  p.N = lo->N; p.C = lo->C; p.XH = lo->H; p.XW = lo->W; p.YH = hi->H; p.YW = hi->W; p.scale = scale;
  p.x_row0 = x_row0; p.in_rows_total = in_rows_total; p.y_row0 = y_row0;
  return AD_OK;
}

}  // namespace adk

using namespace adk;

extern "C" int ad_upsample_bilinear_fwd(const ad_tensor4* x, const ad_tensor4* y, uint32_t scale, int32_t x_row0,
                                        uint32_t in_rows_total, uint32_t y_row0, void* stream) {
  UpP p{};
  int st = up_params(x, y, scale, x_row0, in_rows_total, y_row0, p);
  if (st != AD_OK) return st;
  const size_t total = (size_t)p.N * p.C * p.YH * p.YW;
  if (total == 0) return AD_OK;
  p.c_fastest = y->sc == 1 && y->C > 1;
  if (p.c_fastest && x->sc == 1)
    AD_DISPATCH_DTYPE(x->dtype, (upsample_fwd_px_kernel<T><<<grid_for(total / p.C, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  else
    AD_DISPATCH_DTYPE(x->dtype, (upsample_fwd_kernel<T><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  count_launch();
  return launch_status();
}

extern "C" int ad_upsample_bilinear_bwd(const ad_tensor4* dy, const ad_tensor4* dx, uint32_t scale, int32_t x_row0,
                                        uint32_t in_rows_total, uint32_t y_row0, int32_t accumulate, void* stream) {
  UpP p{};
  int st = up_params(dx, dy, scale, x_row0, in_rows_total, y_row0, p);
  if (st != AD_OK) return st;
  const size_t total = (size_t)p.N * p.C * p.XH * p.XW;
  if (total == 0) return AD_OK;
  p.c_fastest = dx->sc == 1 && dx->C > 1;
  p.accumulate = accumulate;
  if (p.c_fastest && dy->sc == 1)
    AD_DISPATCH_DTYPE(dx->dtype, (upsample_bwd_px_kernel<T><<<grid_for(total / p.C * ((p.C + 7) / 8), 256, 16), 256, 0, as_stream(stream)>>>(p)));
  else
    AD_DISPATCH_DTYPE(dx->dtype, (upsample_bwd_kernel<T><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  count_launch();
  return launch_status();
}
