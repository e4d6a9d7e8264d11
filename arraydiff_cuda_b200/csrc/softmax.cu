// NLL loss on probabilities (the reference's two small kernels) and the fused per-pixel
// softmax cross-entropy.  HBM-bound: logits are read once per pass.
//   NCHW: one thread per pixel, the C strided reads of neighbouring threads coalesce.
//   NHWC: one warp per pixel, lanes over channels, max / sum by warp shuffles.
#include "common.cuh"

namespace adk {

__global__ void nll_fwd_kernel(uint32_t C, uint32_t B, const float* __restrict__ y, const uint32_t* __restrict__ label,
                               float* loss) {
  uint32_t b = threadIdx.x + blockDim.x * blockIdx.x;
  if (b < B) loss[b] = -logf(y[label[b] + (size_t)C * b]);
}

__global__ void nll_bwd_kernel(uint32_t C, uint32_t B, const float* __restrict__ y, const uint32_t* __restrict__ label,
                               const float* __restrict__ dloss, float* dx) {
  size_t idx = threadIdx.x + (size_t)blockDim.x * blockIdx.x;
  if (idx >= (size_t)C * B) return;
  uint32_t c = (uint32_t)(idx % C), b = (uint32_t)(idx / C);
  // Integer label compare (the reference converts the label to float first, which is the
  // same for labels below 2^24: src/kernels/softmax.cu:70-72).
  float yi = y[idx], d = dloss[b];
  float t = label[b] == c ? __fsub_rn(yi, 1.0f) : yi;
  dx[idx] = fmaf(d, t, dx[idx]);
}

template <typename T>
__global__ void __launch_bounds__(256) ce_fwd_nchw(uint32_t N, uint32_t C, uint32_t HW, const T* __restrict__ x,
                                                    const uint32_t* __restrict__ label, float* loss,
                                                    unsigned long long* picked) {
  const size_t total = (size_t)N * HW;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t n = i / HW, t = i % HW;
    const T* px = x + n * C * HW + t;
    float m = -INFINITY;
    for (uint32_t c = 0; c < C; ++c) m = fmaxf(m, ld_f(px + (size_t)c * HW));
    float z = 0.f;
    for (uint32_t c = 0; c < C; ++c) z += expf(ld_f(px + (size_t)c * HW) - m);
    const uint32_t l = label[i];
    const size_t li = (n * C + l) * HW + t;
    loss[i] = (logf(z) + m) - ld_f(x + li);
    if (picked) picked[i] = li;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ce_bwd_nchw(uint32_t N, uint32_t C, uint32_t HW, const T* __restrict__ x,
                                                    const uint32_t* __restrict__ label,
                                                    const float* __restrict__ dloss, T* dx, int accumulate) {
  const size_t total = (size_t)N * HW;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t n = i / HW, t = i % HW;
    const T* px = x + n * C * HW + t;
    T* pdx = dx + n * C * HW + t;
    float m = -INFINITY;
    for (uint32_t c = 0; c < C; ++c) m = fmaxf(m, ld_f(px + (size_t)c * HW));
    float z = 0.f;
    for (uint32_t c = 0; c < C; ++c) z += expf(ld_f(px + (size_t)c * HW) - m);
    const float rz = 1.f / z, d = dloss[i];
    const uint32_t l = label[i];
    for (uint32_t c = 0; c < C; ++c) {
      float pr = expf(ld_f(px + (size_t)c * HW) - m) * rz;
      float g = d * (pr - (c == l ? 1.f : 0.f));
      if (accumulate) g += ld_f(pdx + (size_t)c * HW);
      st_f(pdx + (size_t)c * HW, g);
    }
  }
}

template <typename T, bool BWD>
__global__ void __launch_bounds__(256) ce_nhwc(uint32_t C, size_t pixels, const T* __restrict__ x,
                                                const uint32_t* __restrict__ label, float* loss,
                                                unsigned long long* picked, const float* __restrict__ dloss, T* dx,
                                                int accumulate) {
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = ((size_t)gridDim.x * blockDim.x) >> 5;
  for (size_t i = warp; i < pixels; i += nw) {
    const T* px = x + i * C;
    float m = -INFINITY;
    for (uint32_t c = lane; c < C; c += 32) m = fmaxf(m, ld_f(px + c));
    m = warp_max(m);
    float z = 0.f;
    for (uint32_t c = lane; c < C; c += 32) z += expf(ld_f(px + c) - m);
    z = warp_sum(z);
    const uint32_t l = label[i];
    if (!BWD) {
      if (lane == 0) {
        loss[i] = (logf(z) + m) - ld_f(px + l);
        if (picked) picked[i] = i * C + l;
      }
    } else {
      const float rz = 1.f / z, d = dloss[i];
      for (uint32_t c = lane; c < C; c += 32) {
        float g = d * (expf(ld_f(px + c) - m) * rz - (c == l ? 1.f : 0.f));
        if (accumulate) g += ld_f(dx + i * C + c);
        st_f(dx + i * C + c, g);
      }
    }
  }
}

// Few classes (C <= 32, e.g. 19): a block stages 256 consecutive pixels in shared memory with coalesced loads,
// a thread then owns one pixel (class stride C floats: conflict-free for odd C), results leave coalesced again.
template <typename T, bool BWD>
__global__ void __launch_bounds__(256) ce_nhwc_small(uint32_t C, size_t pixels, const T* __restrict__ x,
                                                      const uint32_t* __restrict__ label, float* loss,
                                                      unsigned long long* picked, const float* __restrict__ dloss, T* dx,
                                                      int accumulate) {
  extern __shared__ float ce_sm[];   // [256][C]
  for (size_t p0 = (size_t)blockIdx.x * 256; p0 < pixels; p0 += (size_t)gridDim.x * 256) {
    const uint32_t np = pixels - p0 < 256 ? (uint32_t)(pixels - p0) : 256u, ne = np * C;
    const T* xb = x + p0 * C;
    for (uint32_t e = threadIdx.x; e < ne; e += 256) ce_sm[e] = ld_f(xb + e);
    __syncthreads();
    if (threadIdx.x < np) {
      float* px = ce_sm + threadIdx.x * C;
      const size_t i = p0 + threadIdx.x;
      float m = -INFINITY;
      for (uint32_t c = 0; c < C; ++c) m = fmaxf(m, px[c]);
      float z = 0.f;
      for (uint32_t c = 0; c < C; ++c) z += expf(px[c] - m);
      const uint32_t l = label[i];
      if (!BWD) {
        loss[i] = (logf(z) + m) - px[l];
        if (picked) picked[i] = i * C + l;
      } else {
        const float rz = 1.f / z, d = dloss[i];
        for (uint32_t c = 0; c < C; ++c) px[c] = d * (expf(px[c] - m) * rz - (c == l ? 1.f : 0.f));
      }
    }
    if (BWD) {
      __syncthreads();
      T* db = dx + p0 * C;
      for (uint32_t e = threadIdx.x; e < ne; e += 256) st_f(db + e, accumulate ? ce_sm[e] + ld_f(db + e) : ce_sm[e]);
    }
    __syncthreads();
  }
}

}  // namespace adk

using namespace adk;

extern "C" int ad_softmax_nll_loss_fwd(uint32_t C, uint32_t B, const float* y, const uint32_t* label, float* loss,
                                       void* stream) {
  if (B == 0) return AD_OK;
  if (!y || !label || !loss || C == 0) return AD_ERR_BAD_ARG;
  nll_fwd_kernel<<<(B + 255) / 256, 256, 0, as_stream(stream)>>>(C, B, y, label, loss);
  count_launch();
  return launch_status();
}

extern "C" int ad_softmax_nll_loss_bwd(uint32_t C, uint32_t B, const float* y, const uint32_t* label,
                                       const float* dloss, float* dx, void* stream) {
  if (B == 0 || C == 0) return AD_OK;
  if (!y || !label || !dloss || !dx) return AD_ERR_BAD_ARG;
  size_t total = (size_t)C * B;
  nll_bwd_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(C, B, y, label, dloss, dx);
  count_launch();
  return launch_status();
}

extern "C" int ad_softmax_ce_pixel_fwd(int32_t dtype, int32_t layout, uint32_t N, uint32_t C, uint32_t HW,
                                       const void* logits, const uint32_t* label, float* loss, uint64_t* picked,
                                       void* stream) {
  if ((size_t)N * HW == 0) return AD_OK;
  if (!logits || !label || !loss || C == 0 || C > 1024) return AD_ERR_BAD_ARG;
  const size_t pixels = (size_t)N * HW;
  cudaStream_t s = as_stream(stream);
  if (layout == AD_NCHW) {
    AD_DISPATCH_DTYPE(dtype, (ce_fwd_nchw<T><<<grid_for(pixels, 256), 256, 0, s>>>(
                                 N, C, HW, (const T*)logits, label, loss, (unsigned long long*)picked)));
  } else if (layout == AD_NHWC && C <= 32) {
    AD_DISPATCH_DTYPE(dtype, (ce_nhwc_small<T, false><<<grid_for(pixels, 256, 16), 256, 256 * C * sizeof(float), s>>>(
                                 C, pixels, (const T*)logits, label, loss, (unsigned long long*)picked, nullptr,
                                 nullptr, 0)));
  } else if (layout == AD_NHWC) {
    AD_DISPATCH_DTYPE(dtype, (ce_nhwc<T, false><<<grid_for(pixels, 8), 256, 0, s>>>(
                                 C, pixels, (const T*)logits, label, loss, (unsigned long long*)picked, nullptr,
                                 nullptr, 0)));
  } else {
    return AD_ERR_UNSUPPORTED;
  }
  count_launch();
  return launch_status();
}

extern "C" int ad_softmax_ce_pixel_bwd(int32_t dtype, int32_t layout, uint32_t N, uint32_t C, uint32_t HW,
                                       const void* logits, const uint32_t* label, const float* dloss, void* dlogits,
                                       int32_t accumulate, void* stream) {
  if ((size_t)N * HW == 0) return AD_OK;
  if (!logits || !label || !dloss || !dlogits || C == 0 || C > 1024) return AD_ERR_BAD_ARG;
  const size_t pixels = (size_t)N * HW;
  cudaStream_t s = as_stream(stream);
  if (layout == AD_NCHW) {
    AD_DISPATCH_DTYPE(dtype, (ce_bwd_nchw<T><<<grid_for(pixels, 256), 256, 0, s>>>(
                                 N, C, HW, (const T*)logits, label, dloss, (T*)dlogits, accumulate)));
  } else if (layout == AD_NHWC && C <= 32) {
    AD_DISPATCH_DTYPE(dtype, (ce_nhwc_small<T, true><<<grid_for(pixels, 256, 16), 256, 256 * C * sizeof(float), s>>>(
                                 C, pixels, (const T*)logits, label, nullptr, nullptr, dloss, (T*)dlogits,
                                 accumulate)));
  } else if (layout == AD_NHWC) {
    AD_DISPATCH_DTYPE(dtype, (ce_nhwc<T, true><<<grid_for(pixels, 8), 256, 0, s>>>(
                                 C, pixels, (const T*)logits, label, nullptr, nullptr, dloss, (T*)dlogits,
                                 accumulate)));
  } else {
    return AD_ERR_UNSUPPORTED;
  }
  count_launch();
  return launch_status();
}
