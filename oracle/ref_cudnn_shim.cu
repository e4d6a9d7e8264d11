// TEST INFRASTRUCTURE ONLY -- never linked into the product library.
//
// The reference computes convolution, pooling, batch normalisation and softmax by calling cuDNN's
// legacy API (peterhj/arraydiff_cuda src/op.cc).  This shim issues the SAME calls with the SAME
// descriptor set-up as those call sites, on small host tensors, so that the CPU oracle (oracle.c) can be
// pinned to what the reference really computes:
//   convolution   cudnnSetConvolution2dDescriptor(pad | 0 for halo-padded input, stride, dilation,
//                 CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT), NCHW float tensors, KCRS filter
//                 (src/op.cc:1343-1422); cudnnConvolutionForward + cudnnAddTensor (:1577-1610),
//                 BackwardBias (:1642-1647), BackwardFilter (:1661-1683), BackwardData (:1702-1724),
//                 algorithms from cudnnFindConvolution*Algorithm as in :1462-1510
//   pooling       cudnnSetPooling2dDescriptor(MAX | AVERAGE_COUNT_INCLUDE_PADDING, NOT_PROPAGATE_NAN,
//                 window, pad 0 over the padded dims, stride) (:3440-3446); Forward (:3496-3513), Backward (:3610-3631)
//   batch norm    CUDNN_BATCHNORM_SPATIAL, epsilon 1e-5, factor 1.0 (:3961-4003); Backward (:4083-4097)
//   softmax       CUDNN_SOFTMAX_ACCURATE, MODE_INSTANCE (:4145-4152) and MODE_CHANNEL (:4216-4223)
// The reference ran on V100 with cuDNN 7, where CUDNN_DATA_FLOAT convolutions are plain fp32 FMA; on
// later GPUs the default math type may route fp32 through TF32 tensor cores, so the convolution descriptor
// is set to CUDNN_FMA_MATH to keep the reference's arithmetic.
//
// Every function takes HOST pointers, allocates what it needs on the current device, runs, copies the
// results back and frees; returns 0 or the line number of the failing call (negated).
#include <cuda_runtime.h>
#include <cudnn.h>
#include <stdint.h>
#include <stdio.h>

#include <vector>

#define CK(x)                                                                                   \
  do {                                                                                          \
    if ((x) != cudaSuccess) { fprintf(stderr, "cuda error at %s:%d\n", __FILE__, __LINE__); return -__LINE__; } \
  } while (0)
#define CD(x)                                                                                    \
  do {                                                                                           \
    cudnnStatus_t s_ = (x);                                                                      \
    if (s_ != CUDNN_STATUS_SUCCESS) {                                                            \
      fprintf(stderr, "cudnn error %s at %s:%d\n", cudnnGetErrorString(s_), __FILE__, __LINE__); \
      return -__LINE__;                                                                          \
    }                                                                                            \
  } while (0)

namespace {
struct Dev {
  std::vector<void*> ptrs;
  ~Dev() { for (void* p : ptrs) cudaFree(p); }
  float* up(const float* h, size_t n) {
    float* d = nullptr;
    if (cudaMalloc(&d, n * sizeof(float) + 16) != cudaSuccess) return nullptr;
    ptrs.push_back(d);
    if (h) cudaMemcpy(d, h, n * sizeof(float), cudaMemcpyHostToDevice);
    else cudaMemset(d, 0, n * sizeof(float));
    return d;
  }
};
int down(float* h, const float* d, size_t n) {
  if (!h) return 0;
  return cudaMemcpy(h, d, n * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}
cudnnHandle_t handle() {
  static cudnnHandle_t h = nullptr;
  if (!h && cudnnCreate(&h) != CUDNN_STATUS_SUCCESS) h = nullptr;
  return h;
}
}  // namespace

extern "C" {

// x [N][C][H][W] as read (padded dims when halo_padded, then `pad` is ignored as the reference does);
// w [K][C][kh][kw]; bias [K] or NULL; dy [N][K][P][Q].  Outputs (any may be NULL): y, dx, dw, db.
int refcudnn_conv(int N, int C, int H, int W, int K, int kh, int kw, int stride, int dil, int pad, int halo_padded,
                  const float* x, const float* w, const float* bias, const float* dy, float* y, float* dx, float* dw,
                  float* db, int* P_out, int* Q_out) {
  cudnnHandle_t h = handle();
  if (!h) return -1;
  cudnnConvolutionDescriptor_t conv;
  cudnnFilterDescriptor_t wd;
  cudnnTensorDescriptor_t xd, yd, bd;
  CD(cudnnCreateConvolutionDescriptor(&conv));
  const int p = halo_padded ? 0 : pad;
  CD(cudnnSetConvolution2dDescriptor(conv, p, p, stride, stride, dil, dil, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT));
  CD(cudnnSetConvolutionMathType(conv, CUDNN_FMA_MATH));
  CD(cudnnCreateFilterDescriptor(&wd));
  CD(cudnnSetFilter4dDescriptor(wd, CUDNN_DATA_FLOAT, CUDNN_TENSOR_NCHW, K, C, kh, kw));
  CD(cudnnCreateTensorDescriptor(&bd));
  CD(cudnnSetTensor4dDescriptor(bd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, 1, K, 1, 1));
  CD(cudnnCreateTensorDescriptor(&xd));
  CD(cudnnSetTensor4dDescriptor(xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  int yn, yc, yh, yw;
  CD(cudnnGetConvolution2dForwardOutputDim(conv, xd, wd, &yn, &yc, &yh, &yw));
  if (P_out) *P_out = yh;
  if (Q_out) *Q_out = yw;
  CD(cudnnCreateTensorDescriptor(&yd));
  CD(cudnnSetTensor4dDescriptor(yd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, yn, yc, yh, yw));
  const size_t nx = (size_t)N * C * H * W, ny = (size_t)yn * yc * yh * yw, nw = (size_t)K * C * kh * kw;
  Dev dev;
  float *dx_ = dev.up(x, nx), *dw_ = dev.up(w, nw), *dy_ = dev.up(nullptr, ny);
  if (!dx_ || !dw_ || !dy_) return -2;
  const float one = 1.f, zero = 0.f;
  int cnt = 0;
  if (y) {
    cudnnConvolutionFwdAlgoPerf_t perf;
    CD(cudnnFindConvolutionForwardAlgorithm(h, xd, wd, conv, yd, 1, &cnt, &perf));
    CD(perf.status);
    void* ws = nullptr;
    if (perf.memory) { CK(cudaMalloc(&ws, perf.memory)); dev.ptrs.push_back(ws); }
    CD(cudnnConvolutionForward(h, &one, xd, dx_, wd, dw_, conv, perf.algo, ws, perf.memory, &zero, yd, dy_));
    if (bias) {
      float* b_ = dev.up(bias, K);
      CD(cudnnAddTensor(h, &one, bd, b_, &one, yd, dy_));
    }
    CK(cudaDeviceSynchronize());
    if (down(y, dy_, ny)) return -3;
  }
  if (dy && (dx || dw || db)) {
    float* g_ = dev.up(dy, ny);
    if (!g_) return -2;
    if (db) {
      float* r_ = dev.up(nullptr, K);
      CD(cudnnConvolutionBackwardBias(h, &one, yd, g_, &zero, bd, r_));
      CK(cudaDeviceSynchronize());
      if (down(db, r_, K)) return -3;
    }
    if (dw) {
      cudnnConvolutionBwdFilterAlgoPerf_t perf;
      CD(cudnnFindConvolutionBackwardFilterAlgorithm(h, xd, yd, conv, wd, 1, &cnt, &perf));
      CD(perf.status);
      void* ws = nullptr;
      if (perf.memory) { CK(cudaMalloc(&ws, perf.memory)); dev.ptrs.push_back(ws); }
      float* r_ = dev.up(nullptr, nw);
      CD(cudnnConvolutionBackwardFilter(h, &one, xd, dx_, yd, g_, conv, perf.algo, ws, perf.memory, &zero, wd, r_));
      CK(cudaDeviceSynchronize());
      if (down(dw, r_, nw)) return -3;
    }
    if (dx) {
      cudnnConvolutionBwdDataAlgoPerf_t perf;
      CD(cudnnFindConvolutionBackwardDataAlgorithm(h, wd, yd, conv, xd, 1, &cnt, &perf));
      CD(perf.status);
      void* ws = nullptr;
      if (perf.memory) { CK(cudaMalloc(&ws, perf.memory)); dev.ptrs.push_back(ws); }
      float* r_ = dev.up(nullptr, nx);
      CD(cudnnConvolutionBackwardData(h, &one, wd, dw_, yd, g_, conv, perf.algo, ws, perf.memory, &zero, xd, r_));
      CK(cudaDeviceSynchronize());
      if (down(dx, r_, nx)) return -3;
    }
  }
  cudnnDestroyTensorDescriptor(xd); cudnnDestroyTensorDescriptor(yd); cudnnDestroyTensorDescriptor(bd);
  cudnnDestroyFilterDescriptor(wd); cudnnDestroyConvolutionDescriptor(conv);
  return 0;
}

// Pooling over explicitly padded dims (descriptor pad 0).  average != 0: CUDNN_POOLING_AVERAGE_COUNT_INCLUDE_PADDING.
int refcudnn_pool(int N, int C, int H, int W, int kh, int kw, int stride, int average, const float* x, const float* dy,
                  float* y, float* dx) {
  cudnnHandle_t h = handle();
  if (!h) return -1;
  cudnnPoolingDescriptor_t pd;
  cudnnTensorDescriptor_t xd, yd;
  CD(cudnnCreatePoolingDescriptor(&pd));
  CD(cudnnSetPooling2dDescriptor(pd, average ? CUDNN_POOLING_AVERAGE_COUNT_INCLUDE_PADDING : CUDNN_POOLING_MAX,
                                 CUDNN_NOT_PROPAGATE_NAN, kh, kw, 0, 0, stride, stride));
  CD(cudnnCreateTensorDescriptor(&xd));
  CD(cudnnSetTensor4dDescriptor(xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  int yn, yc, yh, yw;
  CD(cudnnGetPooling2dForwardOutputDim(pd, xd, &yn, &yc, &yh, &yw));
  CD(cudnnCreateTensorDescriptor(&yd));
  CD(cudnnSetTensor4dDescriptor(yd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, yn, yc, yh, yw));
  const size_t nx = (size_t)N * C * H * W, ny = (size_t)yn * yc * yh * yw;
  Dev dev;
  float *x_ = dev.up(x, nx), *y_ = dev.up(nullptr, ny);
  const float one = 1.f, zero = 0.f;
  CD(cudnnPoolingForward(h, pd, &one, xd, x_, &zero, yd, y_));
  CK(cudaDeviceSynchronize());
  if (down(y, y_, ny)) return -3;
  if (dy && dx) {
    float *g_ = dev.up(dy, ny), *r_ = dev.up(nullptr, nx);
    CD(cudnnPoolingBackward(h, pd, &one, yd, y_, yd, g_, xd, x_, &zero, xd, r_));
    CK(cudaDeviceSynchronize());
    if (down(dx, r_, nx)) return -3;
  }
  cudnnDestroyTensorDescriptor(xd); cudnnDestroyTensorDescriptor(yd); cudnnDestroyPoolingDescriptor(pd);
  return 0;
}

// Spatial batch norm, training statistics.  Outputs: y, save_mean, save_invvar (cuDNN's saved inverse standard
// deviation), run_mean / run_var (factor 1.0: the batch mean and the UNBIASED batch variance), dx, dgamma, dbeta.
int refcudnn_bn(int N, int C, int H, int W, const float* x, const float* gamma, const float* beta, const float* dy,
                float* y, float* save_mean, float* save_invvar, float* run_mean, float* run_var, float* dx,
                float* dgamma, float* dbeta) {
  cudnnHandle_t h = handle();
  if (!h) return -1;
  cudnnTensorDescriptor_t xd, sd;
  CD(cudnnCreateTensorDescriptor(&xd));
  CD(cudnnSetTensor4dDescriptor(xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  CD(cudnnCreateTensorDescriptor(&sd));
  CD(cudnnSetTensor4dDescriptor(sd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, 1, C, 1, 1));
  const size_t nx = (size_t)N * C * H * W;
  Dev dev;
  float *x_ = dev.up(x, nx), *y_ = dev.up(nullptr, nx), *g_ = dev.up(gamma, C), *b_ = dev.up(beta, C);
  float *rm = dev.up(nullptr, C), *rv = dev.up(nullptr, C), *sm = dev.up(nullptr, C), *sv = dev.up(nullptr, C);
  const float one = 1.f, zero = 0.f;
  const double factor = 1.0, eps = 1.0e-5;
  CD(cudnnBatchNormalizationForwardTraining(h, CUDNN_BATCHNORM_SPATIAL, &one, &zero, xd, x_, xd, y_, sd, g_, b_, factor, rm, rv,
                                            eps, sm, sv));
  CK(cudaDeviceSynchronize());
  if (down(y, y_, nx) || down(save_mean, sm, C) || down(save_invvar, sv, C) || down(run_mean, rm, C) || down(run_var, rv, C)) return -3;
  if (dy && dx) {
    float *dy_ = dev.up(dy, nx), *dx_ = dev.up(nullptr, nx), *dg = dev.up(nullptr, C), *db = dev.up(nullptr, C);
    CD(cudnnBatchNormalizationBackward(h, CUDNN_BATCHNORM_SPATIAL, &one, &zero, &one, &zero, xd, x_, xd, dy_, xd, dx_, sd, g_, dg, db,
                                       eps, sm, sv));
    CK(cudaDeviceSynchronize());
    if (down(dx, dx_, nx) || down(dgamma, dg, C) || down(dbeta, db, C)) return -3;
  }
  cudnnDestroyTensorDescriptor(xd); cudnnDestroyTensorDescriptor(sd);
  return 0;
}

// Softmax, CUDNN_SOFTMAX_ACCURATE.  channel_mode 0: MODE_INSTANCE over (C,H,W) of each image; 1: MODE_CHANNEL per pixel.
int refcudnn_softmax(int N, int C, int H, int W, int channel_mode, const float* x, float* y) {
  cudnnHandle_t h = handle();
  if (!h) return -1;
  cudnnTensorDescriptor_t xd;
  CD(cudnnCreateTensorDescriptor(&xd));
  CD(cudnnSetTensor4dDescriptor(xd, CUDNN_TENSOR_NCHW, CUDNN_DATA_FLOAT, N, C, H, W));
  const size_t nx = (size_t)N * C * H * W;
  Dev dev;
  float *x_ = dev.up(x, nx), *y_ = dev.up(nullptr, nx);
  const float one = 1.f, zero = 0.f;
  CD(cudnnSoftmaxForward(h, CUDNN_SOFTMAX_ACCURATE, channel_mode ? CUDNN_SOFTMAX_MODE_CHANNEL : CUDNN_SOFTMAX_MODE_INSTANCE, &one, xd,
                         x_, &zero, xd, y_));
  CK(cudaDeviceSynchronize());
  if (down(y, y_, nx)) return -3;
  cudnnDestroyTensorDescriptor(xd);
  return 0;
}

int refcudnn_version(void) { return (int)cudnnGetVersion(); }

}  // extern "C"
