// Packed fp32 array arithmetic, the fused SGD update, and strided ReLU / add / convert.
// All HBM-bound: one read of each input and one write of each output, 16-byte vectors
// where the pointers allow, grid-stride loops sized from the SM count.
#include "common.cuh"

namespace adk {

unsigned long long g_launch_count = 0;
thread_local int g_last_conv_kernel = kConvNone;

// ---------------------------------------------------------------- packed fp32 arrays
// The rounding of each expression is written out (explicit fmaf / __fmul_rn) so that the
// result does not depend on compiler contraction and matches the reference kernels, which
// nvcc compiles with fused multiply-add (src/kernels/array.cu:58-150).
enum ArrOp { kSet, kAdd, kAddScaled, kAddOnline, kScale, kScaleAdd };

template <int OP>
__device__ __forceinline__ float arr_apply(float a, float b, float x, float y) {
  switch (OP) {
    case kSet: return a;
    case kAdd: return __fadd_rn(x, y);
    case kAddScaled: return fmaf(b, y, __fmul_rn(a, x));
    case kAddOnline: return fmaf(a, __fsub_rn(x, y), y);
    case kScale: return __fmul_rn(a, x);
    default: return fmaf(a, x, y);
  }
}

template <int OP>
__global__ void __launch_bounds__(256) arr_kernel(size_t n, float a, float b, const float* __restrict__ x, float* y) {
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nt = (size_t)gridDim.x * blockDim.x;
  const bool vec = (((uintptr_t)y | (uintptr_t)(OP == kSet ? (const float*)y : x)) & 15u) == 0;
  if (vec) {
    const size_t n4 = n / 4;
    for (size_t i = tid; i < n4; i += nt) {
      float4 xv = OP == kSet ? make_float4(0, 0, 0, 0) : reinterpret_cast<const float4*>(x)[i];
      float4 yv = (OP == kSet || OP == kScale) ? make_float4(0, 0, 0, 0) : reinterpret_cast<float4*>(y)[i];
      yv.x = arr_apply<OP>(a, b, xv.x, yv.x); yv.y = arr_apply<OP>(a, b, xv.y, yv.y);
      yv.z = arr_apply<OP>(a, b, xv.z, yv.z); yv.w = arr_apply<OP>(a, b, xv.w, yv.w);
      reinterpret_cast<float4*>(y)[i] = yv;
    }
    for (size_t i = n4 * 4 + tid; i < n; i += nt)
      y[i] = arr_apply<OP>(a, b, OP == kSet ? 0.f : x[i], (OP == kSet || OP == kScale) ? 0.f : y[i]);
  } else {
    for (size_t i = tid; i < n; i += nt)
      y[i] = arr_apply<OP>(a, b, OP == kSet ? 0.f : x[i], (OP == kSet || OP == kScale) ? 0.f : y[i]);
  }
}

template <int OP>
static int arr_launch(size_t n, float a, float b, const float* x, float* y, void* stream) {
  if (n == 0) return AD_OK;
  if (!y || (OP != kSet && !x)) return AD_ERR_BAD_ARG;
  arr_kernel<OP><<<grid_for((n + 3) / 4, 256), 256, 0, as_stream(stream)>>>(n, a, b, x, y);
  count_launch();
  return launch_status();
}

// ---------------------------------------------------------------- fused SGD
__global__ void __launch_bounds__(256) sgd_kernel(size_t n, float* theta, float* g, float* m, float l2, float mu,
                                                  float alpha, float alpha_next, int nesterov,
                                                  __nv_bfloat16* shadow, const int32_t* guard) {
  // a step whose bounded waits ran out worked on stale halo rows or gradients: leave the parameters alone
  if (guard && *guard != 0) return;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nt = (size_t)gridDim.x * blockDim.x;
  const float nmu = __fmul_rn(-alpha_next, mu);
  for (size_t i = tid; i < n; i += nt) {
    float gi = g[i], th = theta[i], mi = m[i];
    // each line is add_scaled(alpha, x, beta): y = fma(beta, y, round(alpha * x))
    if (l2 != 0.f) gi = fmaf(1.0f, gi, __fmul_rn(l2, th));
    mi = fmaf(mu, mi, __fmul_rn(1.0f, gi));
    if (nesterov) {
      th = fmaf(1.0f, th, __fmul_rn(-alpha, gi));
      th = fmaf(1.0f, th, __fmul_rn(nmu, mi));
    } else {
      th = fmaf(1.0f, th, __fmul_rn(-alpha, mi));
    }
    g[i] = gi; m[i] = mi; theta[i] = th;
    if (shadow) shadow[i] = __float2bfloat16_rn(th);
  }
}

// ---------------------------------------------------------------- strided views
struct View {
  char* base;
  long long sn, sc, sy, sx;
};
static View view_of(const ad_tensor4* t) { return View{(char*)t->base, t->sn, t->sc, t->sy, t->sx}; }

// Linear index -> (n,c,y,x) in the order that makes the OUTPUT view's fastest axis the
// fastest thread index (channel-fastest if sc == 1, else x-fastest).
struct Dims { uint32_t N, C, H, W; int c_fastest; };
__device__ __forceinline__ void unpack(const Dims& d, size_t i, uint32_t& n, uint32_t& c, uint32_t& y, uint32_t& x) {
  if (d.c_fastest) {
    c = (uint32_t)(i % d.C); i /= d.C;
    x = (uint32_t)(i % d.W); i /= d.W;
    y = (uint32_t)(i % d.H); n = (uint32_t)(i / d.H);
  } else {
    x = (uint32_t)(i % d.W); i /= d.W;
    y = (uint32_t)(i % d.H); i /= d.H;
    c = (uint32_t)(i % d.C); n = (uint32_t)(i / d.C);
  }
}
__device__ __forceinline__ long long voff(const View& v, uint32_t n, uint32_t c, uint32_t y, uint32_t x) {
  return n * v.sn + c * v.sc + y * v.sy + x * v.sx;
}

enum EwOp { kRelu, kReluBwd, kAdd2, kConvert };

template <int OP, typename TA, typename TB, typename TY>
__global__ void __launch_bounds__(256) ew_kernel(Dims d, View a, View b, View yv, int accumulate) {
  const size_t total = (size_t)d.N * d.C * d.H * d.W;
  const size_t nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t n, c, y, x;
    unpack(d, i, n, c, y, x);
    TY* yp = (TY*)yv.base + voff(yv, n, c, y, x);
    float av = ld_f((const TA*)a.base + voff(a, n, c, y, x));
    float r;
    if (OP == kRelu) r = fmaxf(av, 0.f);
    else if (OP == kConvert) r = av;
    else {
      float bv = ld_f((const TB*)b.base + voff(b, n, c, y, x));
      r = OP == kAdd2 ? av + bv : (av > 0.f ? bv : 0.f);
    }
    if (accumulate) r += ld_f(yp);
    st_f(yp, r);
  }
}


// bf16 channel-fastest views with 8-element-aligned strides: 8 channels (16 bytes) per thread.
__device__ __forceinline__ void ew_unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) { float2 t = __bfloat1622float2(h[j]); f[2 * j] = t.x; f[2 * j + 1] = t.y; }
}
// Element offset of channel group cg of pixel i; evenly spaced pixels need no division.
__device__ __forceinline__ long long ew_pix_off(const View& v, uint32_t i, uint32_t H, uint32_t W) {
  if (v.sy == (long long)W * v.sx && v.sn == (long long)H * v.sy) return (long long)i * v.sx;
  const uint32_t r = i / W, x = i - r * W, n = r / H, y = r - n * H;
  return n * v.sn + y * v.sy + x * v.sx;
}
// G = C/8 channel groups; the launcher guarantees N*H*W*G < 2^31.  Two items per thread and pass.
template <int OP>
__global__ void __launch_bounds__(256) ew_vec_kernel(Dims d, View a, View b, View yv, int accumulate) {
  const uint32_t G = d.C / 8;
  const uint32_t total = d.N * d.H * d.W * G, nt = gridDim.x * blockDim.x;
  constexpr int U = 2;
  for (uint32_t i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += U * nt) {
    uint4 ar[U], br[U], oldr[U];
    uint4* op[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = i0 + u * nt;
      if (i < total) {
        const uint32_t pix = i / G, cg = i - pix * G;
        ar[u] = *(const uint4*)((const __nv_bfloat16*)a.base + ew_pix_off(a, pix, d.H, d.W) + cg * 8);
        if (OP == kAdd2 || OP == kReluBwd) br[u] = *(const uint4*)((const __nv_bfloat16*)b.base + ew_pix_off(b, pix, d.H, d.W) + cg * 8);
        op[u] = (uint4*)((__nv_bfloat16*)yv.base + ew_pix_off(yv, pix, d.H, d.W) + cg * 8);
        if (accumulate) oldr[u] = *op[u];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i0 + u * nt >= total) break;
      float av[8], bv[8], o[8], old[8];
      ew_unpack8(ar[u], av);
      if (OP == kAdd2 || OP == kReluBwd) ew_unpack8(br[u], bv);
      if (accumulate) ew_unpack8(oldr[u], old);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float v;
        if (OP == kRelu) v = fmaxf(av[j], 0.f);
        else if (OP == kConvert) v = av[j];
        else if (OP == kAdd2) v = av[j] + bv[j];
        else v = av[j] > 0.f ? bv[j] : 0.f;
        o[j] = accumulate ? v + old[j] : v;
      }
      uint4 pk;
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
      *op[u] = pk;
    }
  }
}
static bool ew_vec_ok(const ad_tensor4* t) {
  return t->dtype == AD_BF16 && t->sc == 1 && (t->C & 7u) == 0 && !((uintptr_t)t->base & 15u) && !(t->sn & 7) &&
         !(t->sy & 7) && !(t->sx & 7);
}

static int same_dims(const ad_tensor4* a, const ad_tensor4* b) {
  return a->N == b->N && a->C == b->C && a->H == b->H && a->W == b->W;
}

template <int OP>
static int ew_launch(const ad_tensor4* a, const ad_tensor4* b, const ad_tensor4* y, int accumulate, void* stream) {
  if (!a || !y || !a->base || !y->base || (OP != kRelu && OP != kConvert && (!b || !b->base))) return AD_ERR_BAD_ARG;
  if (!same_dims(a, y) || (b && !same_dims(b, y))) return AD_ERR_BAD_ARG;
  const size_t total = (size_t)y->N * y->C * y->H * y->W;
  if (total == 0) return AD_OK;
  Dims d{y->N, y->C, y->H, y->W, y->sc == 1 && y->C > 1};
  View va = view_of(a), vb = b ? view_of(b) : View{nullptr, 0, 0, 0, 0}, vy = view_of(y);
  cudaStream_t s = as_stream(stream);
  if (total / 8 < (1ull << 31) && ew_vec_ok(a) && ew_vec_ok(y) && (!b || ew_vec_ok(b))) {
    ew_vec_kernel<OP><<<grid_for(total / 16, 256, 16), 256, 0, s>>>(d, va, vb, vy, accumulate);
    count_launch();
    return launch_status();
  }
  const unsigned grid = grid_for(total, 256, 16);
  const int da = a->dtype, db = b ? b->dtype : a->dtype, dy = y->dtype;
#define EW_CASE(TA_, TB_, TY_) ew_kernel<OP, TA_, TB_, TY_><<<grid, 256, 0, s>>>(d, va, vb, vy, accumulate)
  using bf = __nv_bfloat16;
  if (da == AD_F32 && db == AD_F32 && dy == AD_F32) EW_CASE(float, float, float);
  else if (da == AD_BF16 && db == AD_BF16 && dy == AD_BF16) EW_CASE(bf, bf, bf);
  else if (da == AD_F32 && db == AD_F32 && dy == AD_BF16) EW_CASE(float, float, bf);
  else if (da == AD_BF16 && db == AD_BF16 && dy == AD_F32) EW_CASE(bf, bf, float);
  else return AD_ERR_UNSUPPORTED;
#undef EW_CASE
  count_launch();
  return launch_status();
}

}  // namespace adk

using namespace adk;

extern "C" const char* ad_status_string(int status) {
  switch (status) {
    case AD_OK: return "ok";
    case AD_ERR_BAD_ARG: return "bad argument";
    case AD_ERR_UNSUPPORTED: return "unsupported dtype/layout/shape";
    case AD_ERR_CUDA: return "CUDA launch error";
    case AD_ERR_TIMEOUT: return "bounded device wait timed out";
    case AD_ERR_ALIGN: return "misaligned pointer or pitch";
    case AD_ERR_SCRATCH: return "scratch buffer too small";
    case AD_ERR_LIMIT: return "size exceeds a limit built into the entry point";
    default: return "unknown status";
  }
}

extern "C" int32_t ad_conv2d_last_kernel(void) { return g_last_conv_kernel; }
extern "C" uint64_t ad_launch_count(void) { return __atomic_load_n(&g_launch_count, __ATOMIC_RELAXED); }

extern "C" int ad_array_set_constant(size_t n, float c, float* x, void* stream) {
  return arr_launch<kSet>(n, c, 0.f, nullptr, x, stream);
}
extern "C" int ad_array_add(size_t n, const float* x, float* y, void* stream) {
  return arr_launch<kAdd>(n, 0.f, 0.f, x, y, stream);
}
extern "C" int ad_array_add_scaled(size_t n, float alpha, float beta, const float* x, float* y, void* stream) {
  return arr_launch<kAddScaled>(n, alpha, beta, x, y, stream);
}
extern "C" int ad_array_add_online(size_t n, float alpha, const float* x, float* y, void* stream) {
  return arr_launch<kAddOnline>(n, alpha, 0.f, x, y, stream);
}
extern "C" int ad_array_scale(size_t n, float scale, const float* x, float* y, void* stream) {
  return arr_launch<kScale>(n, scale, 0.f, x, y, stream);
}
extern "C" int ad_array_scale_add(size_t n, float scale, const float* x, float* y, void* stream) {
  return arr_launch<kScaleAdd>(n, scale, 0.f, x, y, stream);
}

extern "C" int ad_fill_zero(void* x, size_t bytes, void* stream) {
  if (bytes == 0) return AD_OK;
  if (!x) return AD_ERR_BAD_ARG;
  // A memset node: runs on the copy/fill path at full HBM write bandwidth, no kernel needed.
  return cudaMemsetAsync(x, 0, bytes, as_stream(stream)) == cudaSuccess ? AD_OK : AD_ERR_CUDA;
}

extern "C" int ad_sgd_step(size_t n, float* theta, float* g, float* m, float l2, float mu, float alpha,
                           float alpha_next, int32_t nesterov, void* bf16_shadow, void* stream) {
  if (n == 0) return AD_OK;
  if (!theta || !g || !m) return AD_ERR_BAD_ARG;
  sgd_kernel<<<grid_for(n, 256), 256, 0, as_stream(stream)>>>(n, theta, g, m, l2, mu, alpha, alpha_next, nesterov,
                                                               (__nv_bfloat16*)bf16_shadow, nullptr);
  count_launch();
  return launch_status();
}
extern "C" int ad_sgd_step_guarded(size_t n, float* theta, float* g, float* m, float l2, float mu, float alpha,
                                   float alpha_next, int32_t nesterov, void* bf16_shadow, const int32_t* status_word,
                                   void* stream) {
  if (n == 0) return AD_OK;
  if (!theta || !g || !m) return AD_ERR_BAD_ARG;
  sgd_kernel<<<grid_for(n, 256), 256, 0, as_stream(stream)>>>(n, theta, g, m, l2, mu, alpha, alpha_next, nesterov,
                                                               (__nv_bfloat16*)bf16_shadow, status_word);
  count_launch();
  return launch_status();
}

extern "C" int ad_relu_fwd(const ad_tensor4* x, const ad_tensor4* y, void* stream) {
  return ew_launch<kRelu>(x, nullptr, y, 0, stream);
}
extern "C" int ad_relu_bwd(const ad_tensor4* x, const ad_tensor4* dy, const ad_tensor4* dx, int32_t accumulate,
                           void* stream) {
  return ew_launch<kReluBwd>(x, dy, dx, accumulate, stream);
}
extern "C" int ad_add(const ad_tensor4* a, const ad_tensor4* b, const ad_tensor4* y, void* stream) {
  return ew_launch<kAdd2>(a, b, y, 0, stream);
}
extern "C" int ad_convert(const ad_tensor4* src, const ad_tensor4* dst, int32_t accumulate, void* stream) {
  return ew_launch<kConvert>(src, nullptr, dst, accumulate, stream);
}

// ---------------------------------------------------------------- patch matrix for C_in < 8 layers
namespace adk {
template <typename T>
__global__ void __launch_bounds__(256) im2col_kernel(View x, uint32_t N, uint32_t C, uint32_t H, uint32_t W, uint32_t kh,
                                                     uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw,
                                                     uint32_t P, uint32_t Q, __nv_bfloat16* out, uint32_t ldo) {
  const uint32_t cols = kh * kw * C;
  const size_t total = (size_t)N * P * Q * cols, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t col = (uint32_t)(i % cols);
    const size_t pix = i / cols;
    const uint32_t c = col % C, tap = col / C, s = tap % kw, r = tap / kw;
    const uint32_t q = (uint32_t)(pix % Q);
    const size_t rest = pix / Q;
    const uint32_t p = (uint32_t)(rest % P), n = (uint32_t)(rest / P);
    const uint32_t yy = p * sh + r * dh, xx = q * sw + s * dw;
    float v = 0.f;
    if (yy < H && xx < W) v = ld_f((const T*)x.base + voff(x, n, c, yy, xx));
    out[pix * ldo + col] = __float2bfloat16_rn(v);
  }
}
// Same matrix, 8 output columns (one 16-byte store) per thread; columns past kh*kw*C are written as zeros.
template <typename T>
__global__ void __launch_bounds__(256) im2col_vec_kernel(View x, uint32_t N, uint32_t C, uint32_t H, uint32_t W, uint32_t kh,
                                                         uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw,
                                                         uint32_t P, uint32_t Q, __nv_bfloat16* out, uint32_t ldo) {
  const uint32_t cols = kh * kw * C, groups = ldo / 8;
  const size_t total = (size_t)N * P * Q * groups, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t gcol = (uint32_t)(i % groups) * 8;
    const size_t pix = i / groups;
    const uint32_t q = (uint32_t)(pix % Q);
    const size_t rest = pix / Q;
    const uint32_t p = (uint32_t)(rest % P), n = (uint32_t)(rest / P);
    uint32_t c = gcol % C, tap = gcol / C;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      v[j] = 0.f;
      if (gcol + j < cols) {
        const uint32_t s = tap % kw, r = tap / kw;
        const uint32_t yy = p * sh + r * dh, xx = q * sw + s * dw;
        if (yy < H && xx < W) v[j] = ld_f((const T*)x.base + voff(x, n, c, yy, xx));
      }
      if (++c == C) { c = 0; ++tap; }
    }
    uint4 pk;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    *(uint4*)(out + pix * ldo + gcol) = pk;
  }
}
// Same matrix built one output row per block: the kh input rows the row's patches touch are staged in
// shared memory as bf16 (zeros past the tensor's edge), a table maps each column to its offset inside the
// staged rows, and every thread then assembles 16-byte pieces of the output from shared memory.  Each input
// element is fetched from global memory once per output row instead of once per patch that holds it.
template <typename T>
__global__ void __launch_bounds__(256) im2col_row_kernel(View x, uint32_t C, uint32_t H, uint32_t W, uint32_t kh, uint32_t kw,
                                                         uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw, uint32_t P,
                                                         uint32_t Q, __nv_bfloat16* out, uint32_t ldo, uint32_t rowlen) {
  extern __shared__ __align__(16) unsigned char im2col_smem[];
  __nv_bfloat16* rows = (__nv_bfloat16*)im2col_smem;                                    // [kh][rowlen]
  uint32_t* tab = (uint32_t*)(im2col_smem + (((size_t)kh * rowlen * 2 + 15) & ~(size_t)15));  // [ldo]
  const uint32_t p = blockIdx.x % P, n = blockIdx.x / P, cols = kh * kw * C;
  for (uint32_t t = threadIdx.x; t < ldo; t += 256) {
    uint32_t e = 0xffffffffu;
    if (t < cols) { const uint32_t c = t % C, tap = t / C, s = tap % kw, r = tap / kw; e = r * rowlen + s * dw * C + c; }
    tab[t] = e;
  }
  const bool packed = x.sc == 1 && x.sx == (long long)C;
  for (uint32_t r = 0; r < kh; ++r) {
    const uint32_t yy = p * sh + r * dh;
    const T* src = (const T*)x.base + n * x.sn + yy * x.sy;
    for (uint32_t e = threadIdx.x; e < rowlen; e += 256) {
      float v = 0.f;
      if (yy < H) {
        if (packed) { if (e < W * C) v = ld_f(src + e); }
        else { const uint32_t xx = e / C, c = e - xx * C; if (xx < W) v = ld_f(src + xx * x.sx + c * x.sc); }
      }
      rows[r * rowlen + e] = __float2bfloat16_rn(v);
    }
  }
  __syncthreads();
  const uint32_t groups = ldo / 8;
  __nv_bfloat16* orow = out + ((size_t)n * P + p) * Q * ldo;
  const unsigned short* rs = (const unsigned short*)rows;
  for (uint32_t it = threadIdx.x; it < Q * groups; it += 256) {
    const uint32_t q = it / groups, g = it - q * groups, base = q * sw * C;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t e0 = tab[g * 8 + 2 * j], e1 = tab[g * 8 + 2 * j + 1];
      const uint32_t lo = e0 == 0xffffffffu ? 0u : rs[e0 + base], hi = e1 == 0xffffffffu ? 0u : rs[e1 + base];
      w[j] = lo | (hi << 16);
    }
    *(uint4*)(orow + (size_t)q * ldo + g * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}
template <typename T>
static int launch_im2col_row(const View& v, const ad_tensor4* x, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh,
                             uint32_t dw, uint32_t P, uint32_t Q, __nv_bfloat16* out, uint32_t ldo, uint32_t rowlen, size_t smem,
                             cudaStream_t s) {
  auto kern = im2col_row_kernel<T>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return AD_ERR_CUDA;
  }
  kern<<<x->N * P, 256, smem, s>>>(v, x->C, x->H, x->W, kh, kw, sh, sw, dh, dw, P, Q, out, ldo, rowlen);
  return AD_OK;
}
}  // namespace adk

extern "C" int ad_im2col(const ad_tensor4* x, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw,
                         uint32_t P, uint32_t Q, void* out_bf16, uint32_t ldo, void* stream) {
  if (!x || !x->base || !out_bf16 || kh == 0 || kw == 0 || sh == 0 || sw == 0 || dh == 0 || dw == 0) return AD_ERR_BAD_ARG;
  if (ldo < kh * kw * x->C) return AD_ERR_BAD_ARG;
  const size_t total = (size_t)x->N * P * Q * kh * kw * x->C;
  if (total == 0) return AD_OK;
  adk::View v = adk::view_of(x);
  if ((ldo & 7u) == 0 && ((uintptr_t)out_bf16 & 15u) == 0) {
    // staged-row form when the rows of one output row fit shared memory
    const uint32_t rowlen = ((Q - 1) * sw + (kw - 1) * dw + 1) * x->C;
    const size_t smem = (((size_t)kh * rowlen * 2 + 15) & ~(size_t)15) + (size_t)ldo * 4;
    if (smem <= 100 * 1024 && (size_t)x->N * P < (1ull << 31) && (size_t)Q * (ldo / 8) < (1ull << 31)) {
      int st = AD_OK;
      AD_DISPATCH_DTYPE(x->dtype, (st = adk::launch_im2col_row<T>(v, x, kh, kw, sh, sw, dh, dw, P, Q, (__nv_bfloat16*)out_bf16, ldo,
                                                                  rowlen, smem, adk::as_stream(stream))));
      if (st != AD_OK) return st;
      adk::count_launch();
      return adk::launch_status();
    }
    const size_t tv = (size_t)x->N * P * Q * (ldo / 8);
    AD_DISPATCH_DTYPE(x->dtype, (adk::im2col_vec_kernel<T><<<adk::grid_for(tv, 256, 16), 256, 0, adk::as_stream(stream)>>>(
                                    v, x->N, x->C, x->H, x->W, kh, kw, sh, sw, dh, dw, P, Q, (__nv_bfloat16*)out_bf16, ldo)));
    adk::count_launch();
    return adk::launch_status();
  }
  AD_DISPATCH_DTYPE(x->dtype, (adk::im2col_kernel<T><<<adk::grid_for(total, 256, 16), 256, 0, adk::as_stream(stream)>>>(
                                  v, x->N, x->C, x->H, x->W, kh, kw, sh, sw, dh, dw, P, Q, (__nv_bfloat16*)out_bf16, ldo)));
  adk::count_launch();
  return adk::launch_status();
}
