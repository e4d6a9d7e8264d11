/*
 * CPU oracle for the spatially parallel convolution path of arraydiff_cuda.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, as plain scalar C,
 * what the reference computes on this path so that the CUDA kernels can be checked
 * against it.  Only the tests, the smoke check and the benchmark's CPU-baseline leg
 * may load it; the shipped library never links or calls anything in this file.
 *
 * PARITY PINNING.  The reference ships no golden vectors and no numeric tests for
 * this path.  The byte/index operations here (halo exchange, halo reduce, slice,
 * NLL label indexing, packed array arithmetic) are pinned against the reference's
 * own CUDA kernels, compiled unmodified from its sources and run on a GPU: the
 * fixtures under tests/golden/ were produced that way and the GPU tests repeat the
 * comparison live.  Convolution, pooling, batch normalisation and softmax live in
 * cuDNN in the reference (a closed third-party library; the reference names cuDNN
 * 6.0 in README.md:12 and builds against 7.0.5 in Makefile.config:2).  Those
 * functions restate the documented operator definitions at the reference's call
 * sites; for them parity is UNPINNED by any reference output.
 *
 * Conventions.  Tensors are NCHW unless a function says otherwise, x fastest.
 * A "padded strip" is P[n][c][y][x] with y in [0,h+2p), x in [0,W+2p), interior at
 * [p,p+h) x [p,p+W)  (reference: src/op.cc:2556-2571).
 * Sums are carried in double and rounded once to float, so the oracle is closer
 * to the exact result than any fp32 device reduction order.
 *
 * Build: see oracle/Makefile.  With -fopenmp the outer loops run on all cores
 * (the timed CPU baseline); without it everything is single-threaded.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#define ORC_PAR _Pragma("omp parallel for schedule(static)")
#define ORC_PAR2 _Pragma("omp parallel for collapse(2) schedule(static)")
#else
#define ORC_PAR
#define ORC_PAR2
#endif

#define ORC_LAYOUT_NCHW 0
#define ORC_LAYOUT_NHWC 1
#define ORC_DTYPE_F32 0
#define ORC_DTYPE_BF16 1

int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Sets the OpenMP team size for later calls, whatever OMP_NUM_THREADS said when the library was
 * loaded (a process launcher may export OMP_NUM_THREADS=1 to every rank).  No-op without OpenMP. */
void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* ------------------------------------------------------------------ bf16 */

/* Round-to-nearest-even float -> bfloat16 (NaN kept quiet). */
uint16_t orc_f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

float orc_bf16_to_f32(uint16_t h) {
  uint32_t u = ((uint32_t)h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

void orc_cast_f32_to_bf16(size_t n, const float* x, uint16_t* y) {
  ORC_PAR
  for (size_t i = 0; i < n; ++i) y[i] = orc_f32_to_bf16(x[i]);
}

void orc_cast_bf16_to_f32(size_t n, const uint16_t* x, float* y) {
  ORC_PAR
  for (size_t i = 0; i < n; ++i) y[i] = orc_bf16_to_f32(x[i]);
}

/* x <- float(bf16(x)): what a bf16-operand kernel sees of an fp32 tensor. */
void orc_round_to_bf16_inplace(size_t n, float* x) {
  ORC_PAR
  for (size_t i = 0; i < n; ++i) x[i] = orc_bf16_to_f32(orc_f32_to_bf16(x[i]));
}

/* ---------------------------------------------------- halo exchange / reduce */

/* Element offset of (n, c, y, x) inside a padded strip. */
static size_t strip_off(int layout, int p, int W, int h, int C, int n, int c, int y, int x) {
  size_t Wp = (size_t)W + 2 * (size_t)p, Hp = (size_t)h + 2 * (size_t)p;
  if (layout == ORC_LAYOUT_NCHW) return (((size_t)n * C + c) * Hp + y) * Wp + x;
  return (((size_t)n * Hp + y) * Wp + x) * C + c;
}

/*
 * Halo exchange over a 1 x R grid of H-strips.
 * For r < R-1, d < p:  P_r[.., p+h+d, p+x]   = P_{r+1}[.., p+d, p+x]
 * For r > 0,   d < p:  P_r[.., p-1-d, p+x]   = P_{r-1}[.., p+h-1-d, p+x]
 * Interior columns only; W-pad columns, rank 0's top halo and rank R-1's bottom
 * halo are left untouched.
 * Reference: src/kernels/spatial.cu:175-189 (ExchOp offsets), :401-453 (1x2),
 * :512-594 (1x4); host dispatch src/spatial.cc:75-134.  The reference stops at
 * R = 4; the same neighbour rule is applied here for any R.
 * elem_size is 4 (float) or 2 (bfloat16): a pure copy, so bytes are moved.
 */
void orc_halo_exchange(int R, void** bufs, int elem_size, int layout,
                       int p, int W, int h, int C, int N) {
  for (int r = 0; r < R; ++r) {
    char* dst = (char*)bufs[r];
    for (int side = 0; side < 2; ++side) {
      int src_r = side == 0 ? r + 1 : r - 1;
      if (src_r < 0 || src_r >= R) continue;
      const char* src = (const char*)bufs[src_r];
      for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c)
          for (int d = 0; d < p; ++d) {
            int sy = side == 0 ? p + d : p + h - 1 - d;
            int dy = side == 0 ? p + h + d : p - 1 - d;
            for (int x = 0; x < W; ++x) {
              size_t so = strip_off(layout, p, W, h, C, n, c, sy, p + x);
              size_t dof = strip_off(layout, p, W, h, C, n, c, dy, p + x);
              memcpy(dst + dof * elem_size, src + so * elem_size, (size_t)elem_size);
            }
          }
    }
  }
}

/*
 * Halo-gradient accumulate-back.
 * For r < R-1: G_r[.., p+h-1-d, p+x] += G_{r+1}[.., p-1-d, p+x]
 * For r > 0:   G_r[.., p+d,     p+x] += G_{r-1}[.., p+h+d, p+x]
 * Source halo rows are not cleared.  Each destination element receives exactly
 * one addend per side, so the result does not depend on order when h >= 2p.
 * Reference: src/kernels/spatial.cu:191-205 (ReduceOp offsets), :487-510, :625-652;
 * the reference adds with atomicAdd (include/arraydiff/kernels.hh:67-70), which for
 * one addend per element equals a plain add.
 * dtype f32: float add.  dtype bf16: add in float, round to nearest even.
 */
void orc_halo_reduce(int R, void** bufs, int dtype, int layout,
                     int p, int W, int h, int C, int N) {
  for (int r = 0; r < R; ++r) {
    for (int side = 0; side < 2; ++side) {
      int src_r = side == 0 ? r + 1 : r - 1;
      if (src_r < 0 || src_r >= R) continue;
      for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c)
          for (int d = 0; d < p; ++d) {
            int sy = side == 0 ? p - 1 - d : p + h + d;
            int dy = side == 0 ? p + h - 1 - d : p + d;
            for (int x = 0; x < W; ++x) {
              size_t so = strip_off(layout, p, W, h, C, n, c, sy, p + x);
              size_t dof = strip_off(layout, p, W, h, C, n, c, dy, p + x);
              if (dtype == ORC_DTYPE_F32) {
                ((float*)bufs[r])[dof] += ((const float*)bufs[src_r])[so];
              } else {
                uint16_t* D = (uint16_t*)bufs[r];
                const uint16_t* S = (const uint16_t*)bufs[src_r];
                D[dof] = orc_f32_to_bf16(orc_bf16_to_f32(D[dof]) + orc_bf16_to_f32(S[so]));
              }
            }
          }
    }
  }
}

/*
 * The same two operations on a grid of grid_h x grid_w ranks (rank = gy * grid_w + gx), each holding a padded
 * (h + 2p) x (w + 2p) buffer: every rank's halo cells take the value of the interior cell of the neighbour (one of
 * up to 8: sides and corners) that owns that position of the whole tensor; halo cells beyond the tensor are left
 * untouched.  The reference has the W-split 2 x 1 case (src/kernels/spatial.cu:654-768, column offsets
 * Src/Dst{Next,Prev}Width :175-205) and an unlinked 2 x 2 kernel (:782-1021); the rule restated here is the one
 * all of them implement: cell (Y, X) of the whole tensor lives at padded (p + Y - gy*h, p + X - gx*w) of its owner.
 */
static void halo2d_walk(int reduce, int gw, int gh, void** bufs, int elem_or_dtype, int layout, int p, int w, int h, int C, int N) {
  /* the accumulate-back adds in the order row faces, column faces, corners (the order the device uses) */
  for (int phase = 0; phase < (reduce ? 3 : 1); ++phase)
    for (int r = 0; r < gw * gh; ++r) {
      int gy = r / gw, gx = r % gw;
      for (int dy = -1; dy <= 1; ++dy)
        for (int dx = -1; dx <= 1; ++dx) {
          if (!dy && !dx) continue;
          int kind = (dy && dx) ? 2 : (dy ? 0 : 1);
          if (reduce && kind != phase) continue;
          int ny = gy + dy, nx = gx + dx;
          if (ny < 0 || nx < 0 || ny >= gh || nx >= gw) continue;
          int q = ny * gw + nx;
          /* my halo cells on side (dy, dx) <-> the neighbour's interior cells next to the shared edge */
          int y0 = dy < 0 ? 0 : dy > 0 ? p + h : p, cy = dy == 0 ? h : p;
          int x0 = dx < 0 ? 0 : dx > 0 ? p + w : p, cx = dx == 0 ? w : p;
          int qy0 = dy < 0 ? h : dy > 0 ? p : p, qx0 = dx < 0 ? w : dx > 0 ? p : p;
          for (int n = 0; n < N; ++n)
            for (int c = 0; c < C; ++c)
              for (int y = 0; y < cy; ++y)
                for (int x = 0; x < cx; ++x) {
                  size_t mine = strip_off(layout, p, w, h, C, n, c, y0 + y, x0 + x);
                  size_t his = strip_off(layout, p, w, h, C, n, c, qy0 + y, qx0 + x);
                  if (!reduce) {
                    memcpy((char*)bufs[r] + mine * elem_or_dtype, (const char*)bufs[q] + his * elem_or_dtype, (size_t)elem_or_dtype);
                  } else if (elem_or_dtype == ORC_DTYPE_F32) {
                    /* the neighbour's interior edge cell += my halo copy of it */
                    ((float*)bufs[q])[his] += ((const float*)bufs[r])[mine];
                  } else {
                    uint16_t* D = (uint16_t*)bufs[q];
                    const uint16_t* S = (const uint16_t*)bufs[r];
                    D[his] = orc_f32_to_bf16(orc_bf16_to_f32(D[his]) + orc_bf16_to_f32(S[mine]));
                  }
                }
        }
    }
}
void orc_halo2d_exchange(int gw, int gh, void** bufs, int elem_size, int layout, int p, int w, int h, int C, int N) {
  halo2d_walk(0, gw, gh, bufs, elem_size, layout, p, w, h, C, N);
}
void orc_halo2d_reduce(int gw, int gh, void** bufs, int dtype, int layout, int p, int w, int h, int C, int N) {
  halo2d_walk(1, gw, gh, bufs, dtype, layout, p, w, h, C, N);
}

/* ------------------------------------------------------------ slice / pad */

/*
 * dst[n,c,dh+y,dw+x] (=|+=) src[n,c,sh+y,sw+x] over a count_w x count_h window of
 * packed NCHW tensors.  Argument order follows the reference launcher.
 * Reference: src/kernels/slice.cu:12-41 (index form), :43-105 (copy / add).
 */
void orc_slice2d_hw_nchw_packed(int add, uint32_t count_w, uint32_t count_h,
                                uint32_t src_width, uint32_t src_height,
                                uint32_t dst_width, uint32_t dst_height,
                                uint32_t channels, uint32_t batch_size,
                                const float* src, uint32_t src_w_off, uint32_t src_h_off,
                                float* dst, uint32_t dst_w_off, uint32_t dst_h_off) {
  size_t planes = (size_t)channels * batch_size;
  ORC_PAR
  for (size_t nc = 0; nc < planes; ++nc)
    for (uint32_t y = 0; y < count_h; ++y)
      for (uint32_t x = 0; x < count_w; ++x) {
        size_t s = (src_w_off + x) + (size_t)src_width * ((src_h_off + y) + (size_t)src_height * nc);
        size_t d = (dst_w_off + x) + (size_t)dst_width * ((dst_h_off + y) + (size_t)dst_height * nc);
        if (add) dst[d] += src[s]; else dst[d] = src[s];
      }
}

/*
 * Halo pad forward: zero the whole padded buffer, then copy the packed
 * [N][C][h][W] interior in.  Reference: src/op.cc:2574-2640.
 */
void orc_halo_pad_fwd(int p, int W, int h, int C, int N, const float* x, float* y_padded) {
  size_t Wp = W + 2 * p, Hp = h + 2 * p;
  memset(y_padded, 0, sizeof(float) * Wp * Hp * C * N);
  orc_slice2d_hw_nchw_packed(0, W, h, W, h, (uint32_t)Wp, (uint32_t)Hp, C, N, x, 0, 0, y_padded, p, p);
}

/* Halo pad backward: dx += interior(dy_padded).  Reference: src/op.cc:2644-2711. */
void orc_halo_pad_bwd(int p, int W, int h, int C, int N, const float* dy_padded, float* dx) {
  size_t Wp = W + 2 * p, Hp = h + 2 * p;
  orc_slice2d_hw_nchw_packed(1, W, h, (uint32_t)Wp, (uint32_t)Hp, W, h, C, N, dy_padded, p, p, dx, 0, 0);
}

/* ------------------------------------------------------------ convolution */

/*
 * Cross-correlation (no kernel flip), NCHW input, KCRS filter.
 *   y[n,k,q,s] = b[k] + sum_{c,i,j} xz[n,c, q*sh - ph + i*dh, s*sw - pw + j*dw] * w[k,c,i,j]
 * where xz is x with implicit zero padding (ph,pw).  For a halo-padded input pass
 * the padded strip as x with ph = pw = 0, exactly as the reference tells cuDNN
 * (src/op.cc:1354-1362, :1396-1410).  Call site: src/op.cc:1577-1610.
 * bias may be NULL.
 */
void orc_conv2d_fprop(const float* x, const float* w, const float* bias, float* y,
                      int N, int C, int H, int W, int K, int kh, int kw,
                      int sh, int sw, int dh, int dw, int ph, int pw) {
  int P = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  int Q = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  ORC_PAR2
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k)
      for (int q = 0; q < P; ++q)
        for (int s = 0; s < Q; ++s) {
          double acc = bias ? (double)bias[k] : 0.0;
          for (int c = 0; c < C; ++c)
            for (int i = 0; i < kh; ++i) {
              int yy = q * sh - ph + i * dh;
              if (yy < 0 || yy >= H) continue;
              for (int j = 0; j < kw; ++j) {
                int xx = s * sw - pw + j * dw;
                if (xx < 0 || xx >= W) continue;
                acc += (double)x[(((size_t)n * C + c) * H + yy) * W + xx] *
                       (double)w[(((size_t)k * C + c) * kh + i) * kw + j];
              }
            }
          y[(((size_t)n * K + k) * P + q) * Q + s] = (float)acc;
        }
}

/*
 * Data gradient: dx[n,c,yy,xx] += sum_{k,i,j : yy = q*sh-ph+i*dh, xx = s*sw-pw+j*dw}
 * dy[n,k,q,s] * w[k,c,i,j].  Written over the whole (padded) input extent, so halo
 * rows receive gradient.  Call site: src/op.cc:1702-1724 (beta = 1 accumulate).
 */
void orc_conv2d_dgrad(const float* dy, const float* w, float* dx,
                      int N, int C, int H, int W, int K, int kh, int kw,
                      int sh, int sw, int dh, int dw, int ph, int pw) {
  int P = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  int Q = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  ORC_PAR2
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int yy = 0; yy < H; ++yy)
        for (int xx = 0; xx < W; ++xx) {
          double acc = 0.0;
          for (int i = 0; i < kh; ++i) {
            int t = yy + ph - i * dh;
            if (t < 0 || t % sh) continue;
            int q = t / sh;
            if (q >= P) continue;
            for (int j = 0; j < kw; ++j) {
              int u = xx + pw - j * dw;
              if (u < 0 || u % sw) continue;
              int s = u / sw;
              if (s >= Q) continue;
              for (int k = 0; k < K; ++k)
                acc += (double)dy[(((size_t)n * K + k) * P + q) * Q + s] *
                       (double)w[(((size_t)k * C + c) * kh + i) * kw + j];
            }
          }
          dx[(((size_t)n * C + c) * H + yy) * W + xx] += (float)acc;
        }
}

/*
 * Filter and bias gradient: dw[k,c,i,j] += sum_{n,q,s} dy[n,k,q,s] * xz[n,c,..];
 * db[k] += sum dy[n,k,:,:].  Call sites: src/op.cc:1642-1647 (bias),
 * :1661-1683 (filter).  db may be NULL.
 */
void orc_conv2d_wgrad(const float* x, const float* dy, float* dwt, float* db,
                      int N, int C, int H, int W, int K, int kh, int kw,
                      int sh, int sw, int dh, int dw, int ph, int pw) {
  int P = (H + 2 * ph - dh * (kh - 1) - 1) / sh + 1;
  int Q = (W + 2 * pw - dw * (kw - 1) - 1) / sw + 1;
  ORC_PAR2
  for (int k = 0; k < K; ++k)
    for (int c = 0; c < C; ++c)
      for (int i = 0; i < kh; ++i)
        for (int j = 0; j < kw; ++j) {
          double acc = 0.0;
          for (int n = 0; n < N; ++n)
            for (int q = 0; q < P; ++q) {
              int yy = q * sh - ph + i * dh;
              if (yy < 0 || yy >= H) continue;
              for (int s = 0; s < Q; ++s) {
                int xx = s * sw - pw + j * dw;
                if (xx < 0 || xx >= W) continue;
                acc += (double)dy[(((size_t)n * K + k) * P + q) * Q + s] *
                       (double)x[(((size_t)n * C + c) * H + yy) * W + xx];
              }
            }
          dwt[(((size_t)k * C + c) * kh + i) * kw + j] += (float)acc;
        }
  if (db) {
    ORC_PAR
    for (int k = 0; k < K; ++k) {
      double acc = 0.0;
      for (int n = 0; n < N; ++n)
        for (size_t t = 0; t < (size_t)P * Q; ++t) acc += (double)dy[((size_t)n * K + k) * P * Q + t];
      db[k] += (float)acc;
    }
  }
}

/* --------------------------------------------------------------- pooling */

/*
 * Max pooling on an explicitly padded input (descriptor pad 0, as the reference
 * configures cuDNN for halo-padded inputs: src/op.cc:3440-3446).  The pad cells
 * take part in the max with whatever value the buffer holds (0 after halo pad).
 * argmax (optional) receives the flat index y*W+x of the first maximum in scan
 * order (rows, then columns), which is also the element that receives the gradient.
 */
void orc_maxpool2d_fwd(const float* x, float* y, int32_t* argmax,
                       int N, int C, int H, int W, int kh, int kw, int sh, int sw) {
  int P = (H - kh) / sh + 1, Q = (W - kw) / sw + 1;
  size_t planes = (size_t)N * C;
  ORC_PAR
  for (size_t nc = 0; nc < planes; ++nc)
    for (int q = 0; q < P; ++q)
      for (int s = 0; s < Q; ++s) {
        float best = -INFINITY;
        int bi = 0;
        for (int i = 0; i < kh; ++i)
          for (int j = 0; j < kw; ++j) {
            int yy = q * sh + i, xx = s * sw + j;
            float v = x[(nc * H + yy) * W + xx];
            if (v > best || (i == 0 && j == 0)) { best = v; bi = yy * W + xx; }
          }
        y[(nc * P + q) * Q + s] = best;
        if (argmax) argmax[(nc * P + q) * Q + s] = bi;
      }
}

/* dx[argmax] += dy.  Call site: src/op.cc:3610-3631. */
void orc_maxpool2d_bwd(const float* x, const float* dy, float* dx,
                       int N, int C, int H, int W, int kh, int kw, int sh, int sw) {
  int P = (H - kh) / sh + 1, Q = (W - kw) / sw + 1;
  size_t planes = (size_t)N * C;
  ORC_PAR
  for (size_t nc = 0; nc < planes; ++nc)
    for (int q = 0; q < P; ++q)
      for (int s = 0; s < Q; ++s) {
        float best = -INFINITY;
        int bi = 0;
        for (int i = 0; i < kh; ++i)
          for (int j = 0; j < kw; ++j) {
            int yy = q * sh + i, xx = s * sw + j;
            float v = x[(nc * H + yy) * W + xx];
            if (v > best || (i == 0 && j == 0)) { best = v; bi = yy * W + xx; }
          }
        dx[nc * H * W + bi] += dy[(nc * P + q) * Q + s];
      }
}

/* ------------------------------------------------------ batch normalisation */

/*
 * Spatial batch norm, training mode: per-channel mean and biased variance over
 * (N, H, W), y = gamma * (x - mean) * rsqrt(var + eps) + beta.  save_mean and
 * save_invstd are what the backward pass consumes; batch_var is the biased
 * variance.  (cuDNN writes the UNBIASED variance n/(n-1)*var into its running
 * buffer with factor = 1, src/op.cc:3963; callers that need that value scale.)
 * eps = 1e-5 at the call site src/op.cc:3964, :3988-4003.
 */
void orc_bn_fwd_train(const float* x, const float* gamma, const float* beta, float* y,
                      float* save_mean, float* save_invstd, float* batch_var,
                      int N, int C, int HW, float eps, int relu) {
  ORC_PAR
  for (int c = 0; c < C; ++c) {
    double s = 0.0, ss = 0.0;
    size_t cnt = (size_t)N * HW;
    for (int n = 0; n < N; ++n)
      for (int t = 0; t < HW; ++t) s += (double)x[((size_t)n * C + c) * HW + t];
    double mean = s / (double)cnt;
    for (int n = 0; n < N; ++n)
      for (int t = 0; t < HW; ++t) {
        double d = (double)x[((size_t)n * C + c) * HW + t] - mean;
        ss += d * d;
      }
    double var = ss / (double)cnt;
    double invstd = 1.0 / sqrt(var + (double)eps);
    if (save_mean) save_mean[c] = (float)mean;
    if (save_invstd) save_invstd[c] = (float)invstd;
    if (batch_var) batch_var[c] = (float)var;
    for (int n = 0; n < N; ++n)
      for (int t = 0; t < HW; ++t) {
        size_t i = ((size_t)n * C + c) * HW + t;
        double v = (double)gamma[c] * ((double)x[i] - mean) * invstd + (double)beta[c];
        if (relu && v < 0.0) v = 0.0;
        y[i] = (float)v;
      }
  }
}

/*
 * Batch-norm backward (training statistics).  If relu != 0 the incoming dy is
 * first masked by (y > 0) where y is the forward output recomputed from x.
 *   dbeta  += sum dy ; dgamma += sum dy * xhat
 *   dx     += gamma * invstd * (dy - mean(dy) - xhat * mean(dy * xhat))
 * Call site: src/op.cc:4083-4097.
 */
void orc_bn_bwd(const float* x, const float* dy, const float* gamma, const float* beta,
                const float* save_mean, const float* save_invstd,
                float* dx, float* dgamma, float* dbeta,
                int N, int C, int HW, int relu) {
  ORC_PAR
  for (int c = 0; c < C; ++c) {
    double mean = save_mean[c], invstd = save_invstd[c];
    double sdy = 0.0, sdyx = 0.0;
    size_t cnt = (size_t)N * HW;
    for (int n = 0; n < N; ++n)
      for (int t = 0; t < HW; ++t) {
        size_t i = ((size_t)n * C + c) * HW + t;
        double xhat = ((double)x[i] - mean) * invstd;
        double g = dy[i];
        if (relu && (double)gamma[c] * xhat + (double)beta[c] <= 0.0) g = 0.0;
        sdy += g;
        sdyx += g * xhat;
      }
    if (dbeta) dbeta[c] += (float)sdy;
    if (dgamma) dgamma[c] += (float)sdyx;
    double m1 = sdy / (double)cnt, m2 = sdyx / (double)cnt;
    for (int n = 0; n < N; ++n)
      for (int t = 0; t < HW; ++t) {
        size_t i = ((size_t)n * C + c) * HW + t;
        double xhat = ((double)x[i] - mean) * invstd;
        double g = dy[i];
        if (relu && (double)gamma[c] * xhat + (double)beta[c] <= 0.0) g = 0.0;
        dx[i] += (float)((double)gamma[c] * invstd * (g - m1 - xhat * m2));
      }
  }
}

/* ------------------------------------------------------- relu / residual add */

/* Reference: src/op.cc:3104-3110 (fwd), :3177-3185 (bwd, dx += dy * [x > 0]). */
void orc_relu_fwd(size_t n, const float* x, float* y) {
  ORC_PAR
  for (size_t i = 0; i < n; ++i) y[i] = x[i] > 0.0f ? x[i] : 0.0f;
}

void orc_relu_bwd(size_t n, const float* x, const float* dy, float* dx) {
  ORC_PAR
  for (size_t i = 0; i < n; ++i) dx[i] += x[i] > 0.0f ? dy[i] : 0.0f;
}

/* Packed array arithmetic.  Reference: src/kernels/array.cu:58-150.
 * nvcc contracts a*b + c into one fused multiply-add when it compiles the reference
 * (its default -fmad=true), so the rounding of those kernels is that of fmaf below;
 * this file is compiled with -ffp-contract=off so that nothing else is fused. */
/* alpha*x + beta*y as the reference's add_scaled kernel rounds it: the golden vectors
 * recorded from that kernel show round(alpha*x) first, then one fused beta*y + that. */
static inline float orc_add_scaled1(float alpha, float x, float beta, float y) {
  return fmaf(beta, y, alpha * x);
}

void orc_array_add(size_t n, const float* x, float* y) {              /* y += x        :82-93   */
  ORC_PAR
  for (size_t i = 0; i < n; ++i) { float yi = y[i]; y[i] = x[i] + yi; }
}
void orc_array_add_scaled(size_t n, float alpha, float beta, const float* x, float* y) { /* :96-109 */
  ORC_PAR
  for (size_t i = 0; i < n; ++i) { float yi = y[i]; y[i] = orc_add_scaled1(alpha, x[i], beta, yi); }
}
void orc_array_add_online(size_t n, float alpha, const float* x, float* y) {            /* :111-123 */
  ORC_PAR
  for (size_t i = 0; i < n; ++i) { float yi = y[i]; y[i] = fmaf(alpha, x[i] - yi, yi); }
}
void orc_array_scale(size_t n, float scale, const float* x, float* y) {                 /* :125-136 */
  ORC_PAR
  for (size_t i = 0; i < n; ++i) y[i] = scale * x[i];
}
void orc_array_scale_add(size_t n, float scale, const float* x, float* y) {             /* :138-150 */
  ORC_PAR
  for (size_t i = 0; i < n; ++i) { float yi = y[i]; y[i] = fmaf(scale, x[i], yi); }
}

/* ------------------------------------------------------ softmax / losses */

/*
 * NLL loss on precomputed probabilities, [batch][channels] row-major:
 *   loss[b] = -logf(y[label[b] + C*b]).   Reference: src/kernels/softmax.cu:36-54.
 */
void orc_softmax_nll_loss_fwd(uint32_t C, uint32_t B, const float* y, const uint32_t* label, float* loss) {
  for (uint32_t b = 0; b < B; ++b) loss[b] = -logf(y[label[b] + (size_t)C * b]);
}

/*
 * dx[b,c] += dloss[b] * (y[b,c] - [c == label[b]]).  Reference: src/kernels/softmax.cu:56-78
 * (the reference routes the label through a float; exact below 2^24).
 */
void orc_softmax_nll_loss_bwd(uint32_t C, uint32_t B, const float* y, const uint32_t* label,
                              const float* dloss, float* dx) {
  for (uint32_t b = 0; b < B; ++b)
    for (uint32_t c = 0; c < C; ++c) {
      size_t i = (size_t)C * b + c;
      /* one fused multiply-add per element, as nvcc compiles the reference kernel */
      if (label[b] == c) dx[i] = fmaf(dloss[b], y[i] - 1.0f, dx[i]);
      else dx[i] = fmaf(dloss[b], y[i], dx[i]);
    }
}

/*
 * Per-pixel softmax cross-entropy over NCHW logits [N][C][HW] with labels [N][HW]
 * (softmax over the channel axis, cuDNN's CHANNEL mode that the reference selects
 * at src/op.cc:4216-4223 before asserting "unimplemented" at :4225).
 * prob (optional) gets the softmax; loss[n,t] = -log prob[n,label,t];
 * picked (optional) gets the flat element index of the selected logit.
 */
void orc_softmax_ce_pixel_fwd(const float* logits, const uint32_t* label, float* prob, float* loss,
                              uint64_t* picked, int N, int C, int HW) {
  ORC_PAR
  for (int n = 0; n < N; ++n)
    for (int t = 0; t < HW; ++t) {
      double m = -INFINITY;
      for (int c = 0; c < C; ++c) {
        double v = logits[((size_t)n * C + c) * HW + t];
        if (v > m) m = v;
      }
      double z = 0.0;
      for (int c = 0; c < C; ++c) z += exp((double)logits[((size_t)n * C + c) * HW + t] - m);
      uint32_t l = label[(size_t)n * HW + t];
      size_t li = ((size_t)n * C + l) * HW + t;
      if (prob)
        for (int c = 0; c < C; ++c) {
          size_t i = ((size_t)n * C + c) * HW + t;
          prob[i] = (float)(exp((double)logits[i] - m) / z);
        }
      loss[(size_t)n * HW + t] = (float)(-((double)logits[li] - m - log(z)));
      if (picked) picked[(size_t)n * HW + t] = li;
    }
}

/* dlogits[n,c,t] += dloss[n,t] * (prob[n,c,t] - [c == label[n,t]]) */
void orc_softmax_ce_pixel_bwd(const float* logits, const uint32_t* label, const float* dloss,
                              float* dlogits, int N, int C, int HW) {
  ORC_PAR
  for (int n = 0; n < N; ++n)
    for (int t = 0; t < HW; ++t) {
      double m = -INFINITY;
      for (int c = 0; c < C; ++c) {
        double v = logits[((size_t)n * C + c) * HW + t];
        if (v > m) m = v;
      }
      double z = 0.0;
      for (int c = 0; c < C; ++c) z += exp((double)logits[((size_t)n * C + c) * HW + t] - m);
      uint32_t l = label[(size_t)n * HW + t];
      for (int c = 0; c < C; ++c) {
        size_t i = ((size_t)n * C + c) * HW + t;
        double pr = exp((double)logits[i] - m) / z;
        dlogits[i] += (float)((double)dloss[(size_t)n * HW + t] * (pr - ((uint32_t)c == l ? 1.0 : 0.0)));
      }
    }
}

/* ------------------------------------------------------------ upsampling */

/* Source coordinate for an output index, half-pixel centres (align_corners = false). */
static void bilin_src(int o, int scale, int in_size, int* i0, int* i1, double* f) {
  double src = ((double)o + 0.5) / (double)scale - 0.5;
  if (src < 0.0) src = 0.0;
  int a = (int)floor(src);
  if (a > in_size - 1) a = in_size - 1;
  int b = a + 1 < in_size ? a + 1 : in_size - 1;
  *i0 = a; *i1 = b; *f = src - (double)a;
}

/* Bilinear x`scale` upsample of [planes][H][W] (not present in the reference; used by
 * the segmentation head of the 1024x2048 benchmark configuration). */
void orc_upsample_bilinear_fwd(const float* x, float* y, int planes, int H, int W, int scale) {
  int OH = H * scale, OW = W * scale;
  ORC_PAR
  for (int pl = 0; pl < planes; ++pl)
    for (int oy = 0; oy < OH; ++oy) {
      int y0, y1; double fy;
      bilin_src(oy, scale, H, &y0, &y1, &fy);
      for (int ox = 0; ox < OW; ++ox) {
        int x0, x1; double fx;
        bilin_src(ox, scale, W, &x0, &x1, &fx);
        const float* X = x + (size_t)pl * H * W;
        double v = (1 - fy) * ((1 - fx) * X[y0 * W + x0] + fx * X[y0 * W + x1]) +
                   fy * ((1 - fx) * X[y1 * W + x0] + fx * X[y1 * W + x1]);
        y[((size_t)pl * OH + oy) * OW + ox] = (float)v;
      }
    }
}

void orc_upsample_bilinear_bwd(const float* dy, float* dx, int planes, int H, int W, int scale) {
  int OH = H * scale, OW = W * scale;
  ORC_PAR
  for (int pl = 0; pl < planes; ++pl) {
    double* acc = (double*)calloc((size_t)H * W, sizeof(double));
    for (int oy = 0; oy < OH; ++oy) {
      int y0, y1; double fy;
      bilin_src(oy, scale, H, &y0, &y1, &fy);
      for (int ox = 0; ox < OW; ++ox) {
        int x0, x1; double fx;
        bilin_src(ox, scale, W, &x0, &x1, &fx);
        double g = dy[((size_t)pl * OH + oy) * OW + ox];
        acc[y0 * W + x0] += (1 - fy) * (1 - fx) * g;
        acc[y0 * W + x1] += (1 - fy) * fx * g;
        acc[y1 * W + x0] += fy * (1 - fx) * g;
        acc[y1 * W + x1] += fy * fx * g;
      }
    }
    for (int i = 0; i < H * W; ++i) dx[(size_t)pl * H * W + i] += (float)acc[i];
    free(acc);
  }
}

/* ------------------------------------------------------------------ SGD */

/*
 * One parameter update of the reference's parallel SGD on a flat fp32 buffer,
 * in the reference's operation order (include/arraydiff/optimize.hh:479-499):
 *   g  = l2 * theta + g            (only if l2 != 0)
 *   m  = g + mu * m
 *   nesterov:  theta = -alpha * g + theta ;  theta = -(alpha_next * mu) * m + theta
 *   plain:     theta = -alpha * m + theta
 * Each line is one add_scaled call (alpha*x + beta*y, src/kernels/array.cu:96-109)
 * and is rounded as that kernel rounds.
 */
void orc_sgd_step(size_t n, float* theta, float* g, float* m,
                  float l2, float mu, float alpha, float alpha_next, int nesterov) {
  ORC_PAR
  for (size_t i = 0; i < n; ++i) {
    float gi = g[i], th = theta[i], mi = m[i];
    if (l2 != 0.0f) gi = orc_add_scaled1(l2, th, 1.0f, gi);
    mi = orc_add_scaled1(1.0f, gi, mu, mi);
    if (nesterov) {
      th = orc_add_scaled1(-alpha, gi, 1.0f, th);
      th = orc_add_scaled1(-alpha_next * mu, mi, 1.0f, th);
    } else {
      th = orc_add_scaled1(-alpha, mi, 1.0f, th);
    }
    g[i] = gi; m[i] = mi; theta[i] = th;
  }
}

/* ------------------------------------------------------ layout helpers */

void orc_nchw_to_nhwc(const float* x, float* y, int N, int C, int H, int W) {
  ORC_PAR
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int t = 0; t < H * W; ++t)
        y[((size_t)n * H * W + t) * C + c] = x[((size_t)n * C + c) * H * W + t];
}

void orc_nhwc_to_nchw(const float* x, float* y, int N, int C, int H, int W) {
  ORC_PAR
  for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
      for (int t = 0; t < H * W; ++t)
        y[((size_t)n * C + c) * H * W + t] = x[((size_t)n * H * W + t) * C + c];
}
