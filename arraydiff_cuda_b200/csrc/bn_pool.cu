// Spatial batch normalisation (training statistics, optional fused ReLU) and max pooling
// on strided 4-D views.  HBM-bound.
//
// Statistics are a two-stage, order-fixed reduction: stage 1 writes per-split partial sums
// to caller scratch, stage 2 combines them in double.  No atomics, so results are
// reproducible run to run.  Threads walk the tensor along its fastest axis (x for
// NCHW-like views, channel for NHWC-like views) so that warps read whole sectors.
#include <atomic>

#include "common.cuh"

namespace adk {

constexpr int kBnMaxSplits = 128;
// Partial-sum rows a reduction may use for C channels: as many as fit the scratch of the widest layer
// ((128 + 1) rows of 2 * 2048 floats) beside the two trailing rows (combined sums, their means), at
// most 1024 -- narrow layers get more blocks in flight.
__host__ __device__ inline int bn_max_splits(uint32_t C) {
  long long s = (long long)(kBnMaxSplits + 1) * 2 * 2048 / (2ll * (C ? C : 1)) - 2;
  return (int)(s > 1024 ? 1024 : (s < 1 ? 1 : s));
}

struct BView { const char* base; long long sn, sc, sy, sx; };
static BView bview(const ad_tensor4* t) { return BView{(const char*)t->base, t->sn, t->sc, t->sy, t->sx}; }

// partial[split][0..C) = sum a, partial[split][C..2C) = sum b, where (a, b) is
//   MODE 0: (x, x^2)                      -- forward statistics
//   MODE 1: (g, g * xhat), g = dy masked   -- backward reductions
struct BnRed {
  BView x, dy;
  uint32_t N, C, H, W;
  int relu;
  const float *gamma, *beta, *mean, *invstd;
};

template <typename T, int MODE>
__device__ __forceinline__ void bn_term(const BnRed& p, uint32_t n, uint32_t c, uint32_t y, uint32_t x, float& a,
                                        float& b) {
  const long long ox = n * p.x.sn + c * p.x.sc + y * p.x.sy + x * p.x.sx;
  const float xv = ld_f((const T*)p.x.base + ox);
  if (MODE == 0) {
    a += xv;
    b = fmaf(xv, xv, b);
  } else {
    const long long od = n * p.dy.sn + c * p.dy.sc + y * p.dy.sy + x * p.dy.sx;
    float g = ld_f((const T*)p.dy.base + od);
    const float xhat = (xv - p.mean[c]) * p.invstd[c];
    if (p.relu && fmaf(p.gamma[c], xhat, p.beta[c]) <= 0.f) g = 0.f;
    a += g;
    b = fmaf(g, xhat, b);
  }
}

// NCHW-like: block (256) per (channel, split); threads stride over (n, y, x).
template <typename T, int MODE>
__global__ void __launch_bounds__(256) bn_reduce_xfast(BnRed p, float* partial) {
  const uint32_t c = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const size_t per = (size_t)p.N * p.H * p.W;
  float a = 0.f, b = 0.f;
  for (size_t i = (size_t)split * 256 + threadIdx.x; i < per; i += (size_t)nsplit * 256) {
    uint32_t x = (uint32_t)(i % p.W);
    size_t r = i / p.W;
    uint32_t y = (uint32_t)(r % p.H), n = (uint32_t)(r / p.H);
    bn_term<T, MODE>(p, n, c, y, x, a, b);
  }
  __shared__ float sa[8], sb[8];
  a = warp_sum(a); b = warp_sum(b);
  if ((threadIdx.x & 31) == 0) { sa[threadIdx.x >> 5] = a; sb[threadIdx.x >> 5] = b; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float ta = 0.f, tb = 0.f;
    for (int w = 0; w < 8; ++w) { ta += sa[w]; tb += sb[w]; }
    partial[(size_t)split * 2 * p.C + c] = ta;
    partial[(size_t)split * 2 * p.C + p.C + c] = tb;
  }
}

// NHWC-like: block (32 channels x 8 pixel lanes) per (channel group, split).
template <typename T, int MODE>
__global__ void __launch_bounds__(256) bn_reduce_cfast(BnRed p, float* partial) {
  const uint32_t c = blockIdx.x * 32 + threadIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const size_t per = (size_t)p.N * p.H * p.W;
  float a = 0.f, b = 0.f;
  if (c < p.C)
    for (size_t i = (size_t)split * 8 + threadIdx.y; i < per; i += (size_t)nsplit * 8) {
      uint32_t x = (uint32_t)(i % p.W);
      size_t r = i / p.W;
      uint32_t y = (uint32_t)(r % p.H), n = (uint32_t)(r / p.H);
      bn_term<T, MODE>(p, n, c, y, x, a, b);
    }
  __shared__ float sa[8][33], sb[8][33];
  sa[threadIdx.y][threadIdx.x] = a;
  sb[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y == 0 && c < p.C) {
    float ta = 0.f, tb = 0.f;
    for (int w = 0; w < 8; ++w) { ta += sa[w][threadIdx.x]; tb += sb[w][threadIdx.x]; }
    partial[(size_t)split * 2 * p.C + c] = ta;
    partial[(size_t)split * 2 * p.C + p.C + c] = tb;
  }
}

// Stage 2 of the statistics, 32 channels per block of 1024 threads: 32 row lanes walk the partial rows
// (each warp access is one 128-byte line, up to 8 rows in flight per thread), sum in double, and are
// combined in a fixed order.
//   kind 0: mean / invstd / var from (sum x, sum x^2); double arithmetic for the cancellation in E[x^2]-E[x]^2
//   kind 1: sums[0..2C) = (sum g, sum g*xhat), sums[2C..4C) = those over count; dbeta += sum g, dgamma += sum g*xhat
//   kind 2: sums[0..2C) only
constexpr int kFinishLanes = 32;
__global__ void __launch_bounds__(32 * kFinishLanes) bn_finish(int kind, uint32_t C, int nsplit, const float* __restrict__ partial,
                                                               double count, float eps, float* mean, float* invstd,
                                                               float* var, float* sums, float* dgamma, float* dbeta) {
  const uint32_t lane = threadIdx.x & 31, rl = threadIdx.x >> 5, c = blockIdx.x * 32 + lane;
  double s = 0.0, ss = 0.0;
  if (c < C) {
    for (int k0 = rl; k0 < nsplit; k0 += 8 * kFinishLanes) {
      float v[8], w[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int k = k0 + u * kFinishLanes;
        v[u] = w[u] = 0.f;
        if (k < nsplit) { v[u] = partial[(size_t)k * 2 * C + c]; w[u] = partial[(size_t)k * 2 * C + C + c]; }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) { s += (double)v[u]; ss += (double)w[u]; }
    }
  }
  __shared__ double sh[2][kFinishLanes][33];
  sh[0][rl][lane] = s;
  sh[1][rl][lane] = ss;
  __syncthreads();
  // warp w < 2 sums statistic w: lane = channel, row lanes in order
  if (rl >= 2) return;
  double t = 0.0;
#pragma unroll 8
  for (int w = 0; w < kFinishLanes; ++w) t += sh[rl][w][lane];
  __shared__ double tot[2][32];
  tot[rl][lane] = t;
  __syncwarp();
  // the two warps meet through shared memory: named barrier over these 64 threads
  asm volatile("bar.sync 1, 64;" ::: "memory");
  if (rl != 0 || c >= C) return;
  s = tot[0][lane]; ss = tot[1][lane];
  if (kind == 0) {
    double m = s / count, v = ss / count - m * m;
    if (v < 0.0) v = 0.0;
    if (mean) mean[c] = (float)m;
    if (invstd) invstd[c] = (float)(1.0 / sqrt(v + (double)eps));
    if (var) var[c] = (float)v;
    return;
  }
  const float fs = (float)s, fss = (float)ss;
  sums[c] = fs;
  sums[C + c] = fss;
  if (kind == 1) {
    sums[2 * C + c] = (float)((double)fs / count);
    sums[3 * C + c] = (float)((double)fss / count);
    if (dbeta) dbeta[c] += fs;
    if (dgamma) dgamma[c] += fss;
  }
}

struct BnApply {
  BView x, dy, out;
  uint32_t N, C, H, W;
  int c_fastest, relu, accumulate;
  const float *gamma, *beta, *mean, *invstd;
  const float* partial;  // backward: combined sums [2C], then (vector path) those over count [2C]
  int nsplit;
  double count;
};

// MODE 0: y = relu?(gamma*(x-mean)*invstd+beta)
// MODE 1: dx (+)= gamma*invstd*(g - mean(g) - xhat*mean(g*xhat))
template <typename T, int MODE>
__global__ void __launch_bounds__(256) bn_apply(BnApply p) {
  const size_t total = (size_t)p.N * p.C * p.H * p.W, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, y, x;
    size_t r = i;
    if (p.c_fastest) {
      c = (uint32_t)(r % p.C); r /= p.C; x = (uint32_t)(r % p.W); r /= p.W; y = (uint32_t)(r % p.H); n = (uint32_t)(r / p.H);
    } else {
      x = (uint32_t)(r % p.W); r /= p.W; y = (uint32_t)(r % p.H); r /= p.H; c = (uint32_t)(r % p.C); n = (uint32_t)(r / p.C);
    }
    const float xv = ld_f((const T*)p.x.base + (n * p.x.sn + c * p.x.sc + y * p.x.sy + x * p.x.sx));
    T* op = (T*)p.out.base + (n * p.out.sn + c * p.out.sc + y * p.out.sy + x * p.out.sx);
    const float xhat = (xv - p.mean[c]) * p.invstd[c];
    if (MODE == 0) {
      float v = fmaf(p.gamma[c], xhat, p.beta[c]);
      if (p.relu) v = fmaxf(v, 0.f);
      st_f(op, v);
    } else {
      float g = ld_f((const T*)p.dy.base + (n * p.dy.sn + c * p.dy.sc + y * p.dy.sy + x * p.dy.sx));
      if (p.relu && fmaf(p.gamma[c], xhat, p.beta[c]) <= 0.f) g = 0.f;
      const float m1 = (float)((double)p.partial[c] / p.count), m2 = (float)((double)p.partial[p.C + c] / p.count);
      float v = p.gamma[c] * p.invstd[c] * (g - m1 - xhat * m2);
      if (p.accumulate) v += ld_f(op);
      st_f(op, v);
    }
  }
}


// ------------------------------------------------------------------ NHWC bf16 fast paths
// Channel-fastest bf16 views whose strides are multiples of 8 elements: a thread owns 8 adjacent
// channels (one 16-byte load / store per pixel) of a fixed channel group, so the per-channel
// constants sit in registers and every warp access is a run of whole 128-byte lines.
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(h[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
  return v;
}
// Element offset of pixel i (n, y, x flattened).  Views whose pixels are evenly spaced need no division;
// others decode with 32-bit arithmetic (the launchers require N*H*W < 2^31).
__device__ __forceinline__ long long pix_off(const BView& v, uint32_t i, uint32_t H, uint32_t W) {
  if (v.sy == (long long)W * v.sx && v.sn == (long long)H * v.sy) return (long long)i * v.sx;
  const uint32_t r = i / W, x = i - r * W, n = r / H, y = r - n * H;
  return n * v.sn + y * v.sy + x * v.sx;
}
__device__ __forceinline__ uint4 ld16(const BView& v, long long off) {
  return *(const uint4*)((const __nv_bfloat16*)v.base + off);
}

constexpr int kBnUnroll = 4;  // pixels in flight per thread: all loads of a batch are issued before any use

template <int MODE>
__global__ void __launch_bounds__(256, 2) bn_reduce_vec(BnRed p, float* partial) {
  const uint32_t G = p.C / 8, cg = threadIdx.x % G, pl = threadIdx.x / G, PL = 256 / G;
  const uint32_t per = p.N * p.H * p.W, stride = gridDim.x * PL;
  float a[8], b[8], mean[8], invstd[8], gam[8], bet[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    a[j] = b[j] = 0.f;
    if (MODE == 1) { mean[j] = p.mean[cg * 8 + j]; invstd[j] = p.invstd[cg * 8 + j]; gam[j] = p.gamma[cg * 8 + j]; bet[j] = p.beta[cg * 8 + j]; }
  }
  // Pixels are walked from the last to the first: the tensor was just written front to back by its producer, so its
  // tail is what the L2 still holds; the apply pass that follows walks front to back and meets what this pass read last.
  for (uint32_t i0 = blockIdx.x * PL + pl; i0 < per; i0 += kBnUnroll * stride) {
    uint4 xr[kBnUnroll], gr[kBnUnroll];
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      const uint32_t k = i0 + u * stride;
      if (k < per) {
        const uint32_t i = per - 1u - k;
        xr[u] = ld16(p.x, pix_off(p.x, i, p.H, p.W) + cg * 8);
        if (MODE == 1) gr[u] = ld16(p.dy, pix_off(p.dy, i, p.H, p.W) + cg * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < kBnUnroll; ++u) {
      if (i0 + u * stride >= per) break;
      float xv[8];
      unpack8(xr[u], xv);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { a[j] += xv[j]; b[j] = fmaf(xv[j], xv[j], b[j]); }
      } else {
        float g[8];
        unpack8(gr[u], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = (xv[j] - mean[j]) * invstd[j];
          float gj = g[j];
          if (p.relu && fmaf(gam[j], xhat, bet[j]) <= 0.f) gj = 0.f;
          a[j] += gj;
          b[j] = fmaf(gj, xhat, b[j]);
        }
      }
    }
  }
  __shared__ float sa[256][9], sb[256][9];
#pragma unroll
  for (int j = 0; j < 8; ++j) { sa[threadIdx.x][j] = a[j]; sb[threadIdx.x][j] = b[j]; }
  __syncthreads();
  // thread t < 2C sums one of the block's 2C outputs over the pixel lanes, in lane order
  for (uint32_t t = threadIdx.x; t < 2 * p.C; t += 256) {
    const uint32_t which = t / p.C, c = t - which * p.C, g = c >> 3, j = c & 7;
    float acc = 0.f;
    for (uint32_t q = 0; q < PL; ++q) acc += which ? sb[q * G + g][j] : sa[q * G + g][j];
    partial[(size_t)blockIdx.x * 2 * p.C + t] = acc;
  }
}

// U pixels in flight per thread (the backward form holds three 16-byte values per pixel, so fewer)
template <int MODE, int U = (MODE == 0 ? kBnUnroll : 2)>
__global__ void __launch_bounds__(256, 2) bn_apply_vec(BnApply p) {
  const uint32_t G = p.C / 8, cg = threadIdx.x % G, pl = threadIdx.x / G, PL = 256 / G;
  const uint32_t per = p.N * p.H * p.W, stride = gridDim.x * PL;
  float sc[8], sh[8], mean[8], invstd[8], m1[8], m2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t c = cg * 8 + j;
    mean[j] = p.mean[c]; invstd[j] = p.invstd[c];
    sc[j] = p.gamma[c]; sh[j] = p.beta[c];
    if (MODE == 1) { m1[j] = p.partial[2 * p.C + c]; m2[j] = p.partial[3 * p.C + c]; }
  }
  for (uint32_t i0 = blockIdx.x * PL + pl; i0 < per; i0 += U * stride) {
    uint4 xr[U], gr[U], oldr[U];
    uint4* op[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = i0 + u * stride;
      if (i < per) {
        xr[u] = ld16(p.x, pix_off(p.x, i, p.H, p.W) + cg * 8);
        op[u] = (uint4*)((__nv_bfloat16*)p.out.base + pix_off(p.out, i, p.H, p.W) + cg * 8);
        if (MODE == 1) {
          gr[u] = ld16(p.dy, pix_off(p.dy, i, p.H, p.W) + cg * 8);
          if (p.accumulate) oldr[u] = *op[u];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i0 + u * stride >= per) break;
      float xv[8], o[8];
      unpack8(xr[u], xv);
      if (MODE == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = (xv[j] - mean[j]) * invstd[j];
          float v = fmaf(sc[j], xhat, sh[j]);
          o[j] = p.relu ? fmaxf(v, 0.f) : v;
        }
      } else {
        float g[8], old[8];
        unpack8(gr[u], g);
        if (p.accumulate) unpack8(oldr[u], old);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xhat = (xv[j] - mean[j]) * invstd[j];
          float gj = g[j];
          if (p.relu && fmaf(sc[j], xhat, sh[j]) <= 0.f) gj = 0.f;
          float v = sc[j] * invstd[j] * (gj - m1[j] - xhat * m2[j]);
          o[j] = p.accumulate ? v + old[j] : v;
        }
      }
      *op[u] = pack8(o);
    }
  }
}

static bool vec_view_ok(const ad_tensor4* t) {
  if (t->dtype != AD_BF16 || t->sc != 1 || (t->C & 7u) || t->C < 8 || t->C > 2048) return false;
  if (256 % (t->C / 8)) return false;
  if ((size_t)t->N * t->H * t->W >= (1ull << 31)) return false;
  return !((uintptr_t)t->base & 15u) && !(t->sn & 7) && !(t->sy & 7) && !(t->sx & 7);
}
// blocks of the vector reduction = partial rows: enough to fill the machine, each thread with
// at least one batch of pixels, within the rows the scratch holds
static unsigned vec_grid(const ad_tensor4* t) {
  const size_t per = (size_t)t->N * t->H * t->W, PL = 256 / (t->C / 8);
  size_t g = (per + PL * kBnUnroll - 1) / (PL * kBnUnroll);
  if (g > (size_t)kNumSMs * 2) g = (size_t)kNumSMs * 2;   // two resident blocks per SM keep ~5 MB of loads in flight
  if (g > (size_t)bn_max_splits(t->C)) g = bn_max_splits(t->C);
  return (unsigned)(g < 1 ? 1 : g);
}

static int pick_splits(const ad_tensor4* x, bool cfast) {
  const size_t per = (size_t)x->N * x->H * x->W;
  const size_t groups = cfast ? (x->C + 31) / 32 : x->C;
  size_t want = ((size_t)kNumSMs * 4 + groups - 1) / groups;  // ~4 blocks per SM overall
  size_t maxs = (per + (cfast ? 8 : 256) * 4 - 1) / ((cfast ? 8 : 256) * 4);
  if (want > maxs) want = maxs;
  if (want > (size_t)kBnMaxSplits) want = kBnMaxSplits;
  if (want > (size_t)bn_max_splits(x->C)) want = bn_max_splits(x->C);
  if (want < 1) want = 1;
  return (int)want;
}

template <int MODE>
static int launch_reduce(const BnRed& p, const ad_tensor4* x, float* partial, int& nsplit, cudaStream_t s) {
  const bool cfast = x->sc == 1 && x->C > 1;
  if (vec_view_ok(x) && (MODE == 0 || (p.dy.sc == 1 && !((uintptr_t)p.dy.base & 15u) && !(p.dy.sn & 7) && !(p.dy.sy & 7) && !(p.dy.sx & 7)))) {
    nsplit = (int)vec_grid(x);
    bn_reduce_vec<MODE><<<nsplit, 256, 0, s>>>(p, partial);
    count_launch();
    return launch_status();
  }
  nsplit = pick_splits(x, cfast);
  if (cfast) {
    dim3 grid((x->C + 31) / 32, nsplit), block(32, 8);
    AD_DISPATCH_DTYPE(x->dtype, (bn_reduce_cfast<T, MODE><<<grid, block, 0, s>>>(p, partial)));
  } else {
    dim3 grid(x->C, nsplit);
    AD_DISPATCH_DTYPE(x->dtype, (bn_reduce_xfast<T, MODE><<<grid, 256, 0, s>>>(p, partial)));
  }
  count_launch();
  return launch_status();
}

static bool dims_eq(const ad_tensor4* a, const ad_tensor4* b) {
  return a->N == b->N && a->C == b->C && a->H == b->H && a->W == b->W && a->dtype == b->dtype;
}

// ------------------------------------------------------------------ max pooling
struct PoolP {
  BView x, y, dy, dx;
  uint32_t N, C, H, W, P, Q, kh, kw, sh, sw;
  int c_fastest, accumulate;
};

template <typename T>
__device__ __forceinline__ uint32_t window_argmax(const PoolP& p, uint32_t n, uint32_t c, uint32_t q, uint32_t s, float& best) {
  uint32_t bi = 0;
  best = -INFINITY;
  for (uint32_t i = 0; i < p.kh; ++i)
    for (uint32_t j = 0; j < p.kw; ++j) {
      const uint32_t yy = q * p.sh + i, xx = s * p.sw + j;
      const float v = ld_f((const T*)p.x.base + (n * p.x.sn + c * p.x.sc + yy * p.x.sy + xx * p.x.sx));
      if (v > best || (i == 0 && j == 0)) { best = v; bi = yy * p.W + xx; }
    }
  return bi;
}

template <typename T>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(PoolP p) {
  const size_t total = (size_t)p.N * p.C * p.P * p.Q, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, q, s;
    size_t r = i;
    if (p.c_fastest) {
      c = (uint32_t)(r % p.C); r /= p.C; s = (uint32_t)(r % p.Q); r /= p.Q; q = (uint32_t)(r % p.P); n = (uint32_t)(r / p.P);
    } else {
      s = (uint32_t)(r % p.Q); r /= p.Q; q = (uint32_t)(r % p.P); r /= p.P; c = (uint32_t)(r % p.C); n = (uint32_t)(r / p.C);
    }
    float best;
    window_argmax<T>(p, n, c, q, s, best);
    st_f((T*)p.y.base + (n * p.y.sn + c * p.y.sc + q * p.y.sy + s * p.y.sx), best);
  }
}

// One thread per INPUT element gathers from the windows that contain it; a window
// contributes iff its first maximum is this element.  No atomics -> reproducible.
template <typename T>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(PoolP p) {
  const size_t total = (size_t)p.N * p.C * p.H * p.W, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, y, x;
    size_t r = i;
    if (p.c_fastest) {
      c = (uint32_t)(r % p.C); r /= p.C; x = (uint32_t)(r % p.W); r /= p.W; y = (uint32_t)(r % p.H); n = (uint32_t)(r / p.H);
    } else {
      x = (uint32_t)(r % p.W); r /= p.W; y = (uint32_t)(r % p.H); r /= p.H; c = (uint32_t)(r % p.C); n = (uint32_t)(r / p.C);
    }
    float acc = 0.f;
    // windows q with q*sh <= y <= q*sh + kh - 1
    const uint32_t q_lo = y + 1 > p.kh ? (y + 1 - p.kh + p.sh - 1) / p.sh : 0;
    const uint32_t s_lo = x + 1 > p.kw ? (x + 1 - p.kw + p.sw - 1) / p.sw : 0;
    for (uint32_t q = q_lo; q < p.P && q * p.sh <= y; ++q)
      for (uint32_t s = s_lo; s < p.Q && s * p.sw <= x; ++s) {
        float best;
        if (window_argmax<T>(p, n, c, q, s, best) == y * p.W + x)
          acc += ld_f((const T*)p.dy.base + (n * p.dy.sn + c * p.dy.sc + q * p.dy.sy + s * p.dy.sx));
      }
    T* op = (T*)p.dx.base + (n * p.dx.sn + c * p.dx.sc + y * p.dx.sy + x * p.dx.sx);
    if (p.accumulate) acc += ld_f(op);
    st_f(op, acc);
  }
}


// NHWC bf16 pooling, 8 channels per thread.  Same first-maximum rule as the scalar kernels.
__global__ void __launch_bounds__(256) maxpool_fwd_vec(PoolP p) {
  const uint32_t G = p.C / 8;
  const size_t total = (size_t)p.N * p.P * p.Q * G, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t cg = (uint32_t)(i % G);
    size_t r = i / G;
    const uint32_t s = (uint32_t)(r % p.Q); r /= p.Q;
    const uint32_t q = (uint32_t)(r % p.P), n = (uint32_t)(r / p.P);
    float best[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) best[j] = -INFINITY;
    for (uint32_t a = 0; a < p.kh; ++a)
      for (uint32_t b = 0; b < p.kw; ++b) {
        float v[8];
        unpack8(*(const uint4*)((const __nv_bfloat16*)p.x.base + n * p.x.sn + (q * p.sh + a) * p.x.sy + (s * p.sw + b) * p.x.sx + cg * 8), v);
#pragma unroll
        for (int j = 0; j < 8; ++j) if (v[j] > best[j] || (a == 0 && b == 0)) best[j] = v[j];
      }
    *(uint4*)((__nv_bfloat16*)p.y.base + n * p.y.sn + q * p.y.sy + s * p.y.sx + cg * 8) = pack8(best);
  }
}
// one thread per input pixel x 8 channels; gathers from the (at most ceil(kh/sh) x ceil(kw/sw)) windows over it
__global__ void __launch_bounds__(256) maxpool_bwd_vec(PoolP p) {
  const uint32_t G = p.C / 8;
  const size_t total = (size_t)p.N * p.H * p.W * G, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t cg = (uint32_t)(i % G);
    size_t r = i / G;
    const uint32_t x = (uint32_t)(r % p.W); r /= p.W;
    const uint32_t y = (uint32_t)(r % p.H), n = (uint32_t)(r / p.H);
    const __nv_bfloat16* xb = (const __nv_bfloat16*)p.x.base + n * p.x.sn + cg * 8;
    float acc[8], me[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    unpack8(*(const uint4*)(xb + y * p.x.sy + x * p.x.sx), me);
    const uint32_t q_lo = y + 1 > p.kh ? (y + 1 - p.kh + p.sh - 1) / p.sh : 0;
    const uint32_t s_lo = x + 1 > p.kw ? (x + 1 - p.kw + p.sw - 1) / p.sw : 0;
    for (uint32_t q = q_lo; q < p.P && q * p.sh <= y; ++q)
      for (uint32_t s = s_lo; s < p.Q && s * p.sw <= x; ++s) {
        // this element is the window's first maximum iff no earlier element (scan order) is >= it
        // and no later element is > it
        uint32_t win = 0xffu;   // bit j: channel j of this element is still the window's first maximum
        for (uint32_t a = 0; a < p.kh; ++a)
          for (uint32_t b = 0; b < p.kw; ++b) {
            const uint32_t yy = q * p.sh + a, xx = s * p.sw + b;
            if (yy == y && xx == x) continue;
            float v[8];
            unpack8(*(const uint4*)(xb + yy * p.x.sy + xx * p.x.sx), v);
            const bool earlier = yy < y || (yy == y && xx < x);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (!(earlier ? v[j] < me[j] : v[j] <= me[j])) win &= ~(1u << j);
          }
        float g[8];
        unpack8(*(const uint4*)((const __nv_bfloat16*)p.dy.base + n * p.dy.sn + q * p.dy.sy + s * p.dy.sx + cg * 8), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) if (win & (1u << j)) acc[j] += g[j];
      }
    uint4* op = (uint4*)((__nv_bfloat16*)p.dx.base + n * p.dx.sn + y * p.dx.sy + x * p.dx.sx + cg * 8);
    if (p.accumulate) {
      float old[8];
      unpack8(*op, old);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += old[j];
    }
    *op = pack8(acc);
  }
}
// Tiled backward for NHWC bf16: a block owns a 16 x 16 patch of input pixels for up to 8 channel groups.
// Phase 1 finds, once per window that touches the patch, the position (4 bits per channel) of the window's
// first maximum; phase 2 lets every input pixel pick its gradient from the windows over it.  Same
// first-maximum rule and the same summation order (q, then s, ascending) as the kernels above, with a
// ninth of their loads when windows overlap.
constexpr uint32_t kPoolTile = 16, kPoolMaxWin = 400;
__global__ void __launch_bounds__(256) maxpool_bwd_tile(PoolP p, uint32_t gchunks) {
  __shared__ uint32_t widx[kPoolMaxWin][8];
  const uint32_t G = p.C / 8, gc = blockIdx.x % gchunks, tx = blockIdx.x / gchunks, ty = blockIdx.y, n = blockIdx.z;
  const uint32_t g0 = gc * 8, gcnt = G - g0 < 8 ? G - g0 : 8;
  const uint32_t y0 = ty * kPoolTile, x0 = tx * kPoolTile;
  const uint32_t y1 = y0 + kPoolTile < p.H ? y0 + kPoolTile : p.H, x1 = x0 + kPoolTile < p.W ? x0 + kPoolTile : p.W;
  const uint32_t q_lo = y0 + 1 > p.kh ? (y0 + 1 - p.kh + p.sh - 1) / p.sh : 0;
  const uint32_t s_lo = x0 + 1 > p.kw ? (x0 + 1 - p.kw + p.sw - 1) / p.sw : 0;
  const uint32_t q_hi = (y1 - 1) / p.sh < p.P - 1 ? (y1 - 1) / p.sh : p.P - 1;   // inclusive
  const uint32_t s_hi = (x1 - 1) / p.sw < p.Q - 1 ? (x1 - 1) / p.sw : p.Q - 1;
  const uint32_t nq = q_hi >= q_lo ? q_hi - q_lo + 1 : 0, ns = s_hi >= s_lo ? s_hi - s_lo + 1 : 0;
  const __nv_bfloat16* xb = (const __nv_bfloat16*)p.x.base + n * p.x.sn;
  for (uint32_t it = threadIdx.x; it < nq * ns * gcnt; it += 256) {
    const uint32_t cgl = it % gcnt, w = it / gcnt, s = s_lo + w % ns, q = q_lo + w / ns;
    float best[8];
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) best[j] = -INFINITY;
    for (uint32_t a = 0; a < p.kh; ++a)
      for (uint32_t b = 0; b < p.kw; ++b) {
        float v[8];
        unpack8(*(const uint4*)(xb + (q * p.sh + a) * p.x.sy + (s * p.sw + b) * p.x.sx + (g0 + cgl) * 8), v);
        const uint32_t pos = a * p.kw + b;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (v[j] > best[j] || pos == 0) { best[j] = v[j]; word = (word & ~(15u << (4 * j))) | (pos << (4 * j)); }
      }
    widx[w][cgl] = word;
  }
  __syncthreads();
  const __nv_bfloat16* gb = (const __nv_bfloat16*)p.dy.base + n * p.dy.sn;
  for (uint32_t it = threadIdx.x; it < kPoolTile * kPoolTile * gcnt; it += 256) {
    const uint32_t cgl = it % gcnt, pix = it / gcnt, x = x0 + pix % kPoolTile, y = y0 + pix / kPoolTile;
    if (y >= p.H || x >= p.W) continue;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const uint32_t qa = y + 1 > p.kh ? (y + 1 - p.kh + p.sh - 1) / p.sh : 0;
    const uint32_t sa = x + 1 > p.kw ? (x + 1 - p.kw + p.sw - 1) / p.sw : 0;
    for (uint32_t q = qa; q < p.P && q * p.sh <= y; ++q)
      for (uint32_t s = sa; s < p.Q && s * p.sw <= x; ++s) {
        const uint32_t word = widx[(q - q_lo) * ns + (s - s_lo)][cgl], pos = (y - q * p.sh) * p.kw + (x - s * p.sw);
        float g[8];
        unpack8(*(const uint4*)(gb + q * p.dy.sy + s * p.dy.sx + (g0 + cgl) * 8), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) if (((word >> (4 * j)) & 15u) == pos) acc[j] += g[j];
      }
    uint4* op = (uint4*)((__nv_bfloat16*)p.dx.base + n * p.dx.sn + y * p.dx.sy + x * p.dx.sx + (g0 + cgl) * 8);
    if (p.accumulate) {
      float old[8];
      unpack8(*op, old);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += old[j];
    }
    *op = pack8(acc);
  }
}
// the tile kernel's limits: positions fit 4 bits, the windows over a patch fit its table
static bool pool_tile_ok(const PoolP& p) {
  if (p.kh * p.kw > 16 || p.N > 65535) return false;
  const uint32_t mq = (kPoolTile + p.kh - 2) / p.sh + 1, ms = (kPoolTile + p.kw - 2) / p.sw + 1;
  return mq * ms <= kPoolMaxWin && (p.H + kPoolTile - 1) / kPoolTile <= 65535;
}
static bool pool_vec_ok(const ad_tensor4* t) {
  return t->dtype == AD_BF16 && t->sc == 1 && (t->C & 7u) == 0 && !((uintptr_t)t->base & 15u) && !(t->sn & 7) &&
         !(t->sy & 7) && !(t->sx & 7);
}

}  // namespace adk

using namespace adk;

extern "C" size_t ad_bn_scratch_bytes(uint32_t C) { return (size_t)(bn_max_splits(C) + 2) * 2 * C * sizeof(float); }

extern "C" int ad_bn_partial_stats(const ad_tensor4* x, float* sums, void* scratch, size_t scratch_bytes, void* stream) {
  if (!x || !x->base || !sums || !scratch) return AD_ERR_BAD_ARG;
  if (scratch_bytes < ad_bn_scratch_bytes(x->C)) return AD_ERR_SCRATCH;
  cudaStream_t s = as_stream(stream);
  BnRed p{bview(x), bview(x), x->N, x->C, x->H, x->W, 0, nullptr, nullptr, nullptr, nullptr};
  int nsplit = 1;
  int st = launch_reduce<0>(p, x, (float*)scratch, nsplit, s);
  if (st != AD_OK) return st;
  bn_finish<<<(x->C + 31) / 32, 32 * kFinishLanes, 0, s>>>(2, x->C, nsplit, (const float*)scratch, 1.0, 0.f, nullptr, nullptr, nullptr, sums,
                                             nullptr, nullptr);
  count_launch();
  return launch_status();
}

extern "C" int ad_bn_finalize_apply(const ad_tensor4* x, const ad_tensor4* y, const float* sums, double count,
                                    const float* gamma, const float* beta, float* save_mean, float* save_invstd,
                                    float* batch_var, float eps, int32_t relu, void* stream) {
  if (!x || !y || !x->base || !y->base || !sums || !gamma || !beta || !save_mean || !save_invstd) return AD_ERR_BAD_ARG;
  if (!dims_eq(x, y) || count <= 0.0) return AD_ERR_BAD_ARG;
  cudaStream_t s = as_stream(stream);
  bn_finish<<<(x->C + 31) / 32, 32 * kFinishLanes, 0, s>>>(0, x->C, 1, sums, count, eps, save_mean, save_invstd, batch_var, nullptr, nullptr,
                                             nullptr);
  count_launch();
  BnApply a{bview(x), bview(x), bview(y), x->N, x->C, x->H, x->W, y->sc == 1 && y->C > 1, relu, 0,
            gamma, beta, save_mean, save_invstd, nullptr, 1, count};
  const size_t total = (size_t)x->N * x->C * x->H * x->W;
  if (vec_view_ok(x) && vec_view_ok(y)) bn_apply_vec<0><<<kNumSMs * 4, 256, 0, s>>>(a);
  else AD_DISPATCH_DTYPE(x->dtype, (bn_apply<T, 0><<<grid_for(total, 256, 16), 256, 0, s>>>(a)));
  count_launch();
  return launch_status();
}

extern "C" int ad_bn_fwd_train(const ad_tensor4* x, const ad_tensor4* y, const float* gamma, const float* beta,
                               float* save_mean, float* save_invstd, float* batch_var, float eps, int32_t relu,
                               void* scratch, size_t scratch_bytes, void* stream) {
  if (!x || !y || !x->base || !y->base || !gamma || !beta || !save_mean || !save_invstd || !scratch) return AD_ERR_BAD_ARG;
  if (!dims_eq(x, y)) return AD_ERR_BAD_ARG;
  if (scratch_bytes < ad_bn_scratch_bytes(x->C)) return AD_ERR_SCRATCH;
  const size_t total = (size_t)x->N * x->C * x->H * x->W;
  if (total == 0) return AD_OK;
  cudaStream_t s = as_stream(stream);
  BnRed p{bview(x), bview(x), x->N, x->C, x->H, x->W, 0, nullptr, nullptr, nullptr, nullptr};
  int nsplit = 1;
  int st = launch_reduce<0>(p, x, (float*)scratch, nsplit, s);
  if (st != AD_OK) return st;
  const double count = (double)x->N * x->H * x->W;
  bn_finish<<<(x->C + 31) / 32, 32 * kFinishLanes, 0, s>>>(0, x->C, nsplit, (const float*)scratch, count, eps, save_mean, save_invstd,
                                             batch_var, nullptr, nullptr, nullptr);
  count_launch();
  BnApply a{bview(x), bview(x), bview(y), x->N, x->C, x->H, x->W, y->sc == 1 && y->C > 1, relu, 0,
            gamma, beta, save_mean, save_invstd, nullptr, 1, count};
  if (vec_view_ok(x) && vec_view_ok(y)) bn_apply_vec<0><<<kNumSMs * 4, 256, 0, s>>>(a);
  else AD_DISPATCH_DTYPE(x->dtype, (bn_apply<T, 0><<<grid_for(total, 256, 16), 256, 0, s>>>(a)));
  count_launch();
  return launch_status();
}

// invstd[c] = 1 / sqrt(var[c] + eps), in double as the training path does
__global__ void bn_invstd_kernel(uint32_t C, const float* __restrict__ var, float eps, float* __restrict__ invstd) {
  const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c < C) invstd[c] = (float)(1.0 / sqrt((double)var[c] + (double)eps));
}

extern "C" int ad_bn_fwd_inference(const ad_tensor4* x, const ad_tensor4* y, const float* gamma, const float* beta,
                                   const float* mean, const float* var, float* invstd_out, float eps, int32_t relu,
                                   void* stream) {
  if (!x || !y || !x->base || !y->base || !gamma || !beta || !mean || !var || !invstd_out) return AD_ERR_BAD_ARG;
  if (!dims_eq(x, y)) return AD_ERR_BAD_ARG;
  const size_t total = (size_t)x->N * x->C * x->H * x->W;
  if (total == 0) return AD_OK;
  cudaStream_t s = as_stream(stream);
  bn_invstd_kernel<<<(x->C + 255) / 256, 256, 0, s>>>(x->C, var, eps, invstd_out);
  count_launch();
  BnApply a{bview(x), bview(x), bview(y), x->N, x->C, x->H, x->W, y->sc == 1 && y->C > 1, relu, 0,
            gamma, beta, mean, invstd_out, nullptr, 1, (double)x->N * x->H * x->W};
  if (vec_view_ok(x) && vec_view_ok(y)) bn_apply_vec<0><<<kNumSMs * 4, 256, 0, s>>>(a);
  else AD_DISPATCH_DTYPE(x->dtype, (bn_apply<T, 0><<<grid_for(total, 256, 16), 256, 0, s>>>(a)));
  count_launch();
  return launch_status();
}

extern "C" int ad_bn_bwd(const ad_tensor4* x, const ad_tensor4* dy, const ad_tensor4* dx, const float* gamma,
                         const float* beta, const float* save_mean, const float* save_invstd, float* dgamma,
                         float* dbeta, int32_t relu, int32_t accumulate_dx, void* scratch, size_t scratch_bytes,
                         void* stream) {
  if (!x || !dy || !dx || !x->base || !dy->base || !dx->base || !gamma || !beta || !save_mean || !save_invstd || !scratch)
    return AD_ERR_BAD_ARG;
  if (!dims_eq(x, dy) || !dims_eq(x, dx)) return AD_ERR_BAD_ARG;
  if (scratch_bytes < ad_bn_scratch_bytes(x->C)) return AD_ERR_SCRATCH;
  const size_t total = (size_t)x->N * x->C * x->H * x->W;
  if (total == 0) return AD_OK;
  cudaStream_t s = as_stream(stream);
  BnRed p{bview(x), bview(dy), x->N, x->C, x->H, x->W, relu, gamma, beta, save_mean, save_invstd};
  int nsplit = 1;
  float* partial = (float*)scratch;
  int st = launch_reduce<1>(p, x, partial, nsplit, s);
  if (st != AD_OK) return st;
  float* sums = partial + (size_t)bn_max_splits(x->C) * 2 * x->C;
  const double count = (double)x->N * x->H * x->W;
  bn_finish<<<(x->C + 31) / 32, 32 * kFinishLanes, 0, s>>>(1, x->C, nsplit, partial, count, 0.f, nullptr, nullptr, nullptr, sums, dgamma, dbeta);
  count_launch();
  BnApply a{bview(x), bview(dy), bview(dx), x->N, x->C, x->H, x->W, dx->sc == 1 && dx->C > 1, relu, accumulate_dx,
            gamma, beta, save_mean, save_invstd, sums, 1, count};
  if (vec_view_ok(x) && vec_view_ok(dy) && vec_view_ok(dx)) bn_apply_vec<1><<<kNumSMs * 4, 256, 0, s>>>(a);
  else AD_DISPATCH_DTYPE(x->dtype, (bn_apply<T, 1><<<grid_for(total, 256, 16), 256, 0, s>>>(a)));
  count_launch();
  return launch_status();
}

static int pool_params(const ad_tensor4* x, const ad_tensor4* y, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw,
                       PoolP& p) {
  if (!x || !y || !x->base || !y->base || kh == 0 || kw == 0 || sh == 0 || sw == 0) return AD_ERR_BAD_ARG;
  if (x->H < kh || x->W < kw) return AD_ERR_BAD_ARG;
  const uint32_t P = (x->H - kh) / sh + 1, Q = (x->W - kw) / sw + 1;
  if (y->N != x->N || y->C != x->C || y->H != P || y->W != Q || y->dtype != x->dtype) return AD_ERR_BAD_ARG;
  p.x = bview(x);
  p.N = x->N; p.C = x->C; p.H = x->H; p.W = x->W; p.P = P; p.Q = Q;
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw;
  return AD_OK;
}

extern "C" int ad_maxpool2d_fwd(const ad_tensor4* x, const ad_tensor4* y, uint32_t kh, uint32_t kw, uint32_t sh,
                                uint32_t sw, void* stream) {
  PoolP p{};
  int st = pool_params(x, y, kh, kw, sh, sw, p);
  if (st != AD_OK) return st;
  p.y = bview(y);
  p.c_fastest = y->sc == 1 && y->C > 1;
  const size_t total = (size_t)p.N * p.C * p.P * p.Q;
  if (total == 0) return AD_OK;
  if (pool_vec_ok(x) && pool_vec_ok(y)) maxpool_fwd_vec<<<grid_for(total / 8, 256, 16), 256, 0, as_stream(stream)>>>(p);
  else AD_DISPATCH_DTYPE(x->dtype, (maxpool_fwd_kernel<T><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  count_launch();
  return launch_status();
}

extern "C" int ad_maxpool2d_bwd(const ad_tensor4* x, const ad_tensor4* dy, const ad_tensor4* dx, uint32_t kh,
                                uint32_t kw, uint32_t sh, uint32_t sw, int32_t accumulate, void* stream) {
  PoolP p{};
  int st = pool_params(x, dy, kh, kw, sh, sw, p);
  if (st != AD_OK) return st;
  if (!dx || !dx->base || dx->N != x->N || dx->C != x->C || dx->H != x->H || dx->W != x->W || dx->dtype != x->dtype)
    return AD_ERR_BAD_ARG;
  p.dy = bview(dy);
  p.dx = bview(dx);
  p.c_fastest = dx->sc == 1 && dx->C > 1;
  p.accumulate = accumulate;
  const size_t total = (size_t)p.N * p.C * p.H * p.W;
  if (total == 0) return AD_OK;
  if (pool_vec_ok(x) && pool_vec_ok(dy) && pool_vec_ok(dx) && pool_tile_ok(p)) {
    const uint32_t gchunks = (p.C / 8 + 7) / 8;
    dim3 grid((p.W + kPoolTile - 1) / kPoolTile * gchunks, (p.H + kPoolTile - 1) / kPoolTile, p.N);
    maxpool_bwd_tile<<<grid, 256, 0, as_stream(stream)>>>(p, gchunks);
  } else if (pool_vec_ok(x) && pool_vec_ok(dy) && pool_vec_ok(dx)) maxpool_bwd_vec<<<grid_for(total / 8, 256, 16), 256, 0, as_stream(stream)>>>(p);
  else AD_DISPATCH_DTYPE(x->dtype, (maxpool_bwd_kernel<T><<<grid_for(total, 256, 16), 256, 0, as_stream(stream)>>>(p)));
  count_launch();
  return launch_status();
}

// ------------------------------------------------------------------ allocation-free variant
// Some callers of this library are not in a position to allocate device memory for the
// statistics scratch: an op body running inside a host framework that has handed the whole
// device to its own memory pool, or a latency-critical loop in which cudaMalloc (which may
// synchronise the device) must not appear.  For them the scratch of the batch-norm forward
// lives in this file-scope device array, sized for at most kBnStaticMaxC channels.  The array
// exists once per GPU that loads the library and is held until the process exits.
constexpr uint32_t kBnStaticMaxC = 2048;
constexpr size_t kBnStaticBytes = (size_t)(adk::kBnMaxSplits + 1) * 2 * kBnStaticMaxC * sizeof(float);
static __device__ __align__(256) unsigned char g_bn_static_scratch[kBnStaticBytes];

// In host code the array's name is only a handle for the runtime, never a device address:
// the address has to be asked for, once per device, with that device current.
// The per-device cache is a table of atomics: host threads that make the first call on one device at the
// same time each look the symbol up and store the same value; none can read a half-written pointer.
static int bn_static_scratch_address(void** out) {
  constexpr int kMaxDevices = 64;
  static std::atomic<void*> addr[kMaxDevices];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return AD_ERR_CUDA; }
  void* p = addr[dev].load(std::memory_order_acquire);
  if (!p) {
    if (cudaGetSymbolAddress(&p, g_bn_static_scratch) != cudaSuccess || !p) { cudaGetLastError(); return AD_ERR_CUDA; }
    addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return AD_OK;
}

extern "C" int ad_bn_fwd_train_noalloc(const ad_tensor4* x, const ad_tensor4* y, const float* gamma, const float* beta,
                                       float* save_mean, float* save_invstd, float* batch_var, float eps, int32_t relu,
                                       void* stream) {
  if (!x) return AD_ERR_BAD_ARG;
  if (x->C > kBnStaticMaxC) return AD_ERR_LIMIT;  // more channels than the built-in scratch holds
  void* scratch = nullptr;
  int st = bn_static_scratch_address(&scratch);
  if (st != AD_OK) return st;
  // Every word of the scratch that the kernels read is written earlier in the same call, so
  // nothing has to be cleared even though the array keeps the previous call's contents.
  return ad_bn_fwd_train(x, y, gamma, beta, save_mean, save_invstd, batch_var, eps, relu, scratch, kBnStaticBytes, stream);
}
