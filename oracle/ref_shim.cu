// C entry points over the reference's own CUDA kernel launchers, so that tests can
// run the unmodified reference kernels on a GPU and compare them with the CPU oracle.
// Test infrastructure only.  The reference's sources are compiled where they lie
// (see the Makefile's `ref` target); nothing of them is copied here.
//
// Each function forwards to the launcher named in its comment
// (include/arraydiff/kernels.hh) on the stream given and returns cudaGetLastError().
#include "arraydiff/kernels.hh"

#include <cuda_runtime.h>
#include <cstdint>

using namespace arraydiff;

extern "C" {

// kernels.hh:116-126 / :128-138 ; ranks live in one address space, so the "peer"
// pointers may all point into one GPU's memory.
int ref_halo_1x2(int reduce, uint32_t rank, uint32_t p, uint32_t W, uint32_t h, uint32_t C, uint32_t N,
                 float* x0, float* x1, cudaStream_t s) {
  if (reduce) spatial2d_1x2_halo_reduce_nchw<float>(rank, p, W, h, C, N, x0, x1, s);
  else spatial2d_1x2_halo_exch_nchw<float>(rank, p, W, h, C, N, x0, x1, s);
  return (int)cudaGetLastError();
}

// kernels.hh:140-166
int ref_halo_1x4(int reduce, uint32_t rank, uint32_t p, uint32_t W, uint32_t h, uint32_t C, uint32_t N,
                 float* x0, float* x1, float* x2, float* x3, cudaStream_t s) {
  if (reduce) spatial2d_1x4_halo_reduce_nchw<float>(rank, p, W, h, C, N, x0, x1, x2, x3, s);
  else spatial2d_1x4_halo_exch_nchw<float>(rank, p, W, h, C, N, x0, x1, x2, x3, s);
  return (int)cudaGetLastError();
}

// kernels.hh:168-178: the W-split pair (2 ranks side by side), exchange only -- src/kernels/spatial.cu:654-733.  The
// float specialisation of the matching reduce is declared (:770-780) but never defined, so the reference cannot link
// it; reduce != 0 returns -3.  Callers keep halo_pad * base_height * channels * batch <= 16384 so that the launcher
// picks one block: its per-block work split (total / blocks, rounded up) can run past the end for other block counts.
int ref_halo_2x1(int reduce, uint32_t rank, uint32_t p, uint32_t W, uint32_t h, uint32_t C, uint32_t N,
                 float* x0, float* x1, cudaStream_t s) {
  if (reduce) return -3;
  if ((unsigned long long)p * h * C * N > 16384ull) return -2;
  spatial2d_2x1_halo_exch_nchw<float>(rank, p, W, h, C, N, x0, x1, s);
  return (int)cudaGetLastError();
}

// kernels.hh:222-256
int ref_slice2d(int add, uint32_t count_w, uint32_t count_h, uint32_t src_width, uint32_t src_height,
                uint32_t dst_width, uint32_t dst_height, uint32_t channels, uint32_t batch_size,
                const float* src, uint32_t src_w_off, uint32_t src_h_off,
                float* dst, uint32_t dst_w_off, uint32_t dst_h_off, cudaStream_t s) {
  if (add) slice2d_add_hw_nchw_packed<float>(count_w, count_h, src_width, src_height, dst_width, dst_height,
                                             channels, batch_size, src, src_w_off, src_h_off, dst, dst_w_off, dst_h_off, s);
  else slice2d_copy_hw_nchw_packed<float>(count_w, count_h, src_width, src_height, dst_width, dst_height,
                                          channels, batch_size, src, src_w_off, src_h_off, dst, dst_w_off, dst_h_off, s);
  return (int)cudaGetLastError();
}

// kernels.hh:98-102
int ref_softmax_nll_loss_fwd(uint32_t C, uint32_t B, const float* y, const uint32_t* label, float* loss, cudaStream_t s) {
  softmax_nll_loss_fwd<float>(C, B, y, label, loss, s);
  return (int)cudaGetLastError();
}
int ref_softmax_nll_loss_bwd(uint32_t C, uint32_t B, const float* y, const uint32_t* label, const float* dloss,
                             float* dx, cudaStream_t s) {
  softmax_nll_loss_bwd<float>(C, B, y, label, dloss, dx, s);
  return (int)cudaGetLastError();
}

// kernels.hh:72-93 ; op: 0 add, 1 add_scaled, 2 add_online, 3 scale, 4 scale_add
int ref_array_op(int op, uint32_t n, float a, float b, const float* x, float* y, cudaStream_t s) {
  switch (op) {
    case 0: array_add_packed<float>(n, x, y, s); break;
    case 1: array_add_scaled_packed<float>(n, a, b, x, y, s); break;
    case 2: array_add_online_packed<float>(n, a, x, y, s); break;
    case 3: array_scale_packed<float>(n, a, x, y, s); break;
    case 4: array_scale_add_packed<float>(n, a, x, y, s); break;
    default: return -1;
  }
  return (int)cudaGetLastError();
}

}  // extern "C"
