// Strided row-segment copy / accumulate: the one kernel behind halo exchange, halo-gradient
// accumulate-back, 2-D slicing and halo pad / unpad.
//
// All of these move a set of equally long, contiguous row segments between two strided
// tensors (for NCHW one segment per (plane, row) of W elements; for NHWC one per (image,
// row) of W*C elements).  Each warp takes one chunk (<= 2 KiB) of one segment at a time:
//   * source and destination equally aligned modulo 16 B -> straight 16-byte vector
//     loads/stores with scalar head and tail;
//   * otherwise the chunk is staged through shared memory: 16-byte loads aligned to the
//     source, 16-byte stores aligned to the destination, re-aligned in between.  That
//     keeps both the reads and the writes (the side that crosses NVLink in a halo push)
//     at full vector width even though a padded fp32 row of W+2p elements is in general
//     not a multiple of 16 bytes.
// HBM / NVLink bound; grid is sized in multiples of the SM count.
#include "common.cuh"

namespace adk {

constexpr int kMaxJobs = 2 * AD_MAX_PEERS;
constexpr int kChunk = 2048;            // bytes of one segment handled per warp step
constexpr int kWarpsPerBlock = 8;
constexpr int kStage = kChunk + 32;     // staging bytes per warp (16 B of slack either side)

struct SegJob {
  const char* src;
  char* dst;
  uint32_t src_row0, dst_row0;
  int32_t signal_rank;  // -1: none
  // geometry of this job's segments; zero rows = take the launch-wide values of SegParams (filled in by launch_seg)
  uint32_t rows, seg_bytes, chunks_per_seg;
  uint32_t src_xoff, dst_xoff;         // bytes
  unsigned long long first_unit;       // work units (plane, row, chunk) of the jobs before this one
};

struct SegParams {
  SegJob jobs[kMaxJobs];
  int32_t njobs;
  int32_t elem;         // element size in bytes (4 or 2)
  int32_t accumulate;   // dst += src (fp32 add; bf16: fp32 add + RNE)
  uint32_t planes, rows;
  uint32_t seg_bytes, chunks_per_seg;
  unsigned long long total_units;
  unsigned long long src_plane_stride, src_row_stride, src_xoff;  // bytes
  unsigned long long dst_plane_stride, dst_row_stride, dst_xoff;  // bytes
  // completion signal (halo exchange)
  uint64_t* signal_flags[AD_MAX_PEERS];
  uint32_t signal_mask;
  uint64_t epoch;
  const unsigned long long* epoch_base;
  uint32_t* block_counter;
};

template <int ELEM> struct ElemT;
template <> struct ElemT<4> { using type = uint32_t; };
template <> struct ElemT<2> { using type = uint16_t; };

template <int ELEM>
__device__ __forceinline__ typename ElemT<ELEM>::type add_elem(typename ElemT<ELEM>::type d,
                                                               typename ElemT<ELEM>::type s) {
  if (ELEM == 4) {
    return __float_as_uint(__uint_as_float(d) + __uint_as_float(s));
  } else {
    float fd = __uint_as_float(((uint32_t)d) << 16), fs = __uint_as_float(((uint32_t)s) << 16);
    __nv_bfloat16 r = __float2bfloat16_rn(fd + fs);
    return (typename ElemT<ELEM>::type)__bfloat16_as_ushort(r);
  }
}

__device__ __forceinline__ uint4 add_vec(uint4 d, uint4 s, int elem) {
  uint4 r;
  if (elem == 4) {
    r.x = add_elem<4>(d.x, s.x); r.y = add_elem<4>(d.y, s.y);
    r.z = add_elem<4>(d.z, s.z); r.w = add_elem<4>(d.w, s.w);
  } else {
    uint32_t* dp = &d.x; uint32_t* sp = &s.x; uint32_t* rp = &r.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint32_t lo = add_elem<2>((uint16_t)(dp[i] & 0xffffu), (uint16_t)(sp[i] & 0xffffu));
      uint32_t hi = add_elem<2>((uint16_t)(dp[i] >> 16), (uint16_t)(sp[i] >> 16));
      rp[i] = lo | (hi << 16);
    }
  }
  return r;
}

// Moves `len` bytes (a multiple of ELEM) from s to d with one warp.
template <int ELEM, bool ACC>
__device__ __forceinline__ void warp_move(const char* __restrict__ s, char* __restrict__ d, uint32_t len,
                                          char* stage, int lane) {
  using E = typename ElemT<ELEM>::type;
  const uint32_t sa = (uint32_t)((uintptr_t)s & 15u), da = (uint32_t)((uintptr_t)d & 15u);
  if (sa == da) {
    // Same phase: head up to the first 16-byte boundary, vector body, scalar tail.
    uint32_t head = (16u - sa) & 15u;
    if (head > len) head = len;
    for (uint32_t o = lane * ELEM; o < head; o += 32 * ELEM) {
      E v = *(const E*)(s + o);
      if (ACC) v = add_elem<ELEM>(*(E*)(d + o), v);
      *(E*)(d + o) = v;
    }
    const uint32_t body = (len - head) & ~15u;
    for (uint32_t o = head + lane * 16; o < head + body; o += 32 * 16) {
      uint4 v = *(const uint4*)(s + o);
      if (ACC) v = add_vec(*(uint4*)(d + o), v, ELEM);
      *(uint4*)(d + o) = v;
    }
    for (uint32_t o = head + body + lane * ELEM; o < len; o += 32 * ELEM) {
      E v = *(const E*)(s + o);
      if (ACC) v = add_elem<ELEM>(*(E*)(d + o), v);
      *(E*)(d + o) = v;
    }
    return;
  }
  // Different phase: stage[sa + k] holds byte k of the segment.
  {
    uint32_t head = (16u - sa) & 15u;
    if (head > len) head = len;
    for (uint32_t o = lane * ELEM; o < head; o += 32 * ELEM) *(E*)(stage + sa + o) = *(const E*)(s + o);
    const uint32_t body = (len - head) & ~15u;
    for (uint32_t o = head + lane * 16; o < head + body; o += 32 * 16)
      *(uint4*)(stage + sa + o) = *(const uint4*)(s + o);  // sa + head is a multiple of 16
    for (uint32_t o = head + body + lane * ELEM; o < len; o += 32 * ELEM)
      *(E*)(stage + sa + o) = *(const E*)(s + o);
  }
  __syncwarp();
  {
    const char* st = stage + sa;
    uint32_t head = (16u - da) & 15u;
    if (head > len) head = len;
    for (uint32_t o = lane * ELEM; o < head; o += 32 * ELEM) {
      E v = *(const E*)(st + o);
      if (ACC) v = add_elem<ELEM>(*(E*)(d + o), v);
      *(E*)(d + o) = v;
    }
    const uint32_t body = (len - head) & ~15u;
    for (uint32_t o = head + lane * 16; o < head + body; o += 32 * 16) {
      uint4 v;
      if (ELEM == 4) {
        v.x = *(const uint32_t*)(st + o); v.y = *(const uint32_t*)(st + o + 4);
        v.z = *(const uint32_t*)(st + o + 8); v.w = *(const uint32_t*)(st + o + 12);
      } else {
        uint32_t* vp = &v.x;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          vp[i] = (uint32_t)*(const uint16_t*)(st + o + 4 * i) | ((uint32_t)*(const uint16_t*)(st + o + 4 * i + 2) << 16);
      }
      if (ACC) v = add_vec(*(uint4*)(d + o), v, ELEM);
      *(uint4*)(d + o) = v;
    }
    for (uint32_t o = head + body + lane * ELEM; o < len; o += 32 * ELEM) {
      E v = *(const E*)(st + o);
      if (ACC) v = add_elem<ELEM>(*(E*)(d + o), v);
      *(E*)(d + o) = v;
    }
  }
  __syncwarp();
}

template <int ELEM, bool ACC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) seg_move_kernel(const SegParams prm) {
  __shared__ __align__(16) char stage_all[kWarpsPerBlock][kStage];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  char* stage = stage_all[warp];
  const unsigned long long total = prm.total_units;
  const unsigned long long nwarps = (unsigned long long)gridDim.x * kWarpsPerBlock;
  for (unsigned long long u = (unsigned long long)blockIdx.x * kWarpsPerBlock + warp; u < total; u += nwarps) {
    uint32_t job = 0;
    while (job + 1 < (uint32_t)prm.njobs && u >= prm.jobs[job + 1].first_unit) ++job;
    const SegJob& jb = prm.jobs[job];
    unsigned long long r = u - jb.first_unit;
    const uint32_t chunk = (uint32_t)(r % jb.chunks_per_seg);
    r /= jb.chunks_per_seg;
    const uint32_t row = (uint32_t)(r % jb.rows);
    const unsigned long long plane = r / jb.rows;
    const uint32_t off = chunk * kChunk;
    uint32_t len = jb.seg_bytes - off;
    if (len > (uint32_t)kChunk) len = kChunk;
    const char* s = jb.src + plane * prm.src_plane_stride + (unsigned long long)(jb.src_row0 + row) * prm.src_row_stride +
                    jb.src_xoff + off;
    char* d = jb.dst + plane * prm.dst_plane_stride + (unsigned long long)(jb.dst_row0 + row) * prm.dst_row_stride +
              jb.dst_xoff + off;
    warp_move<ELEM, ACC>(s, d, len, stage, lane);
  }
  if (prm.signal_mask != 0u) {
    // Publish: every thread's remote stores are ordered (system scope) before the block's
    // ticket; the block that takes the last ticket releases the flags.
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned ticket = atomicAdd(prm.block_counter, 1u);
      if (ticket == gridDim.x - 1) {
        __threadfence_system();
        *prm.block_counter = 0u;
        const unsigned long long value = (unsigned long long)prm.epoch + (prm.epoch_base ? *prm.epoch_base : 0ull);
        for (int q = 0; q < AD_MAX_PEERS; ++q)
          if (prm.signal_mask & (1u << q)) {
            unsigned long long* f = (unsigned long long*)prm.signal_flags[q];
            asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(f), "l"(value) : "memory");
          }
      }
    }
  }
}

static int launch_seg(SegParams& prm, cudaStream_t stream) {
  unsigned long long total = 0;
  for (int j = 0; j < prm.njobs; ++j) {
    SegJob& jb = prm.jobs[j];
    if (jb.rows == 0) {      // a job without its own geometry takes the launch-wide one
      jb.rows = prm.rows; jb.seg_bytes = prm.seg_bytes;
      jb.src_xoff = (uint32_t)prm.src_xoff; jb.dst_xoff = (uint32_t)prm.dst_xoff;
    }
    jb.chunks_per_seg = (jb.seg_bytes + kChunk - 1) / kChunk;
    jb.first_unit = total;
    total += (unsigned long long)prm.planes * jb.rows * jb.chunks_per_seg;
  }
  prm.total_units = total;
  if (total == 0) return AD_OK;
  const unsigned grid = grid_for((size_t)total, kWarpsPerBlock, 8);
  dim3 block(kWarpsPerBlock * 32);
  if (prm.elem == 4) {
    if (prm.accumulate) seg_move_kernel<4, true><<<grid, block, 0, stream>>>(prm);
    else seg_move_kernel<4, false><<<grid, block, 0, stream>>>(prm);
  } else {
    if (prm.accumulate) seg_move_kernel<2, true><<<grid, block, 0, stream>>>(prm);
    else seg_move_kernel<2, false><<<grid, block, 0, stream>>>(prm);
  }
  count_launch();
  return launch_status();
}

static int check_halo(const ad_halo_args* a) {
  if (!a) return AD_ERR_BAD_ARG;
  if (elem_size(a->dtype) == 0) return AD_ERR_UNSUPPORTED;
  if (a->layout != AD_NCHW && a->layout != AD_NHWC) return AD_ERR_UNSUPPORTED;
  if (a->num_ranks < 1 || a->num_ranks > AD_MAX_PEERS) return AD_ERR_BAD_ARG;
  if (a->rank_first + a->rank_count > a->num_ranks || a->rank_count == 0) return AD_ERR_BAD_ARG;
  if (a->base_width == 0 || a->base_height == 0 || a->num_channels == 0 || a->batch_size == 0) return AD_ERR_BAD_ARG;
  if (a->num_ranks > 1 && a->base_height < 2 * a->halo_pad) return AD_ERR_BAD_ARG;
  for (uint32_t r = 0; r < a->num_ranks; ++r) {
    // Only neighbours of the served ranks are dereferenced, but a null anywhere is a caller bug.
    bool needed = (r + 1 >= a->rank_first && r <= a->rank_first + a->rank_count);
    if (needed && !a->bufs[r]) return AD_ERR_BAD_ARG;
    if (needed && ((uintptr_t)a->bufs[r] % (uintptr_t)elem_size(a->dtype)) != 0) return AD_ERR_ALIGN;
  }
  return AD_OK;
}

static void halo_geometry(const ad_halo_args* a, SegParams& prm) {
  const unsigned long long es = (unsigned long long)elem_size(a->dtype);
  const unsigned long long p = a->halo_pad, W = a->base_width, h = a->base_height, C = a->num_channels,
                           N = a->batch_size;
  const unsigned long long Wp = W + 2 * p, Hp = h + 2 * p;
  prm.elem = (int)es;
  prm.rows = (uint32_t)p;
  if (a->layout == AD_NCHW) {
    prm.planes = (uint32_t)(N * C);
    prm.seg_bytes = (uint32_t)(W * es);
    prm.src_plane_stride = Hp * Wp * es;
    prm.src_row_stride = Wp * es;
    prm.src_xoff = p * es;
  } else {
    prm.planes = (uint32_t)N;
    prm.seg_bytes = (uint32_t)(W * C * es);
    prm.src_plane_stride = Hp * Wp * C * es;
    prm.src_row_stride = Wp * C * es;
    prm.src_xoff = p * C * es;
  }
  prm.dst_plane_stride = prm.src_plane_stride;
  prm.dst_row_stride = prm.src_row_stride;
  prm.dst_xoff = prm.src_xoff;
  prm.chunks_per_seg = (prm.seg_bytes + kChunk - 1) / kChunk;
}

}  // namespace adk

using namespace adk;

extern "C" int ad_halo_exchange(const ad_halo_args* a, void* stream) {
  int st = check_halo(a);
  if (st != AD_OK) return st;
  if (a->halo_pad == 0 || a->num_ranks == 1) return AD_OK;
  SegParams prm{};
  halo_geometry(a, prm);
  const uint32_t p = a->halo_pad, h = a->base_height, R = a->num_ranks;
  bool want_signal = false;
  for (uint32_t q = 0; q < R; ++q) want_signal |= (a->signal_flags[q] != nullptr);
  if (want_signal && !a->block_counter) return AD_ERR_BAD_ARG;
  int nj = 0;
  for (uint32_t r = a->rank_first; r < a->rank_first + a->rank_count; ++r) {
    if (a->push) {
      if (r + 1 < R) prm.jobs[nj++] = SegJob{(const char*)a->bufs[r], (char*)a->bufs[r + 1], h, 0, (int)(r + 1)};
      if (r > 0) prm.jobs[nj++] = SegJob{(const char*)a->bufs[r], (char*)a->bufs[r - 1], p, p + h, (int)(r - 1)};
    } else {
      if (r + 1 < R) prm.jobs[nj++] = SegJob{(const char*)a->bufs[r + 1], (char*)a->bufs[r], p, p + h, (int)r};
      if (r > 0) prm.jobs[nj++] = SegJob{(const char*)a->bufs[r - 1], (char*)a->bufs[r], h, 0, (int)r};
    }
  }
  prm.njobs = nj;
  prm.accumulate = 0;
  if (want_signal) {
    for (int j = 0; j < nj; ++j) {
      int q = prm.jobs[j].signal_rank;
      if (q >= 0 && a->signal_flags[q]) {
        prm.signal_flags[q] = a->signal_flags[q];
        prm.signal_mask |= 1u << q;
      }
    }
    prm.epoch = a->epoch;
    prm.epoch_base = (const unsigned long long*)a->epoch_base;
    prm.block_counter = a->block_counter;
  }
  return launch_seg(prm, as_stream(stream));
}

extern "C" int ad_halo_reduce(const ad_halo_args* a, void* stream) {
  int st = check_halo(a);
  if (st != AD_OK) return st;
  if (a->halo_pad == 0 || a->num_ranks == 1) return AD_OK;
  SegParams prm{};
  halo_geometry(a, prm);
  const uint32_t p = a->halo_pad, h = a->base_height, R = a->num_ranks;
  int nj = 0;
  for (uint32_t r = a->rank_first; r < a->rank_first + a->rank_count; ++r) {
    if (r + 1 < R) prm.jobs[nj++] = SegJob{(const char*)a->bufs[r + 1], (char*)a->bufs[r], 0, h, -1};
    if (r > 0) prm.jobs[nj++] = SegJob{(const char*)a->bufs[r - 1], (char*)a->bufs[r], p + h, p, -1};
  }
  prm.njobs = nj;
  prm.accumulate = 1;
  return launch_seg(prm, as_stream(stream));
}

static int slice2d(int add, int32_t dtype, uint32_t count_w, uint32_t count_h, uint32_t src_width, uint32_t src_height,
                   uint32_t dst_width, uint32_t dst_height, uint32_t channels, uint32_t batch_size, const void* src,
                   uint32_t src_w_off, uint32_t src_h_off, void* dst, uint32_t dst_w_off, uint32_t dst_h_off,
                   void* stream) {
  const unsigned long long es = (unsigned long long)elem_size(dtype);
  if (es == 0) return AD_ERR_UNSUPPORTED;
  if (!src || !dst) return AD_ERR_BAD_ARG;
  if (count_w == 0 || count_h == 0 || channels == 0 || batch_size == 0) return AD_OK;
  if ((unsigned long long)src_w_off + count_w > src_width || (unsigned long long)src_h_off + count_h > src_height ||
      (unsigned long long)dst_w_off + count_w > dst_width || (unsigned long long)dst_h_off + count_h > dst_height)
    return AD_ERR_BAD_ARG;
  if (((uintptr_t)src % es) || ((uintptr_t)dst % es)) return AD_ERR_ALIGN;
  SegParams prm{};
  prm.elem = (int)es;
  prm.accumulate = add;
  prm.njobs = 1;
  prm.jobs[0] = SegJob{(const char*)src, (char*)dst, src_h_off, dst_h_off, -1};
  prm.planes = channels * batch_size;
  prm.rows = count_h;
  prm.seg_bytes = (uint32_t)(count_w * es);
  prm.chunks_per_seg = (prm.seg_bytes + kChunk - 1) / kChunk;
  prm.src_plane_stride = (unsigned long long)src_width * src_height * es;
  prm.src_row_stride = (unsigned long long)src_width * es;
  prm.src_xoff = (unsigned long long)src_w_off * es;
  prm.dst_plane_stride = (unsigned long long)dst_width * dst_height * es;
  prm.dst_row_stride = (unsigned long long)dst_width * es;
  prm.dst_xoff = (unsigned long long)dst_w_off * es;
  return launch_seg(prm, as_stream(stream));
}

extern "C" int ad_slice2d_copy_hw_nchw_packed(int32_t dtype, uint32_t count_w, uint32_t count_h, uint32_t src_width,
                                              uint32_t src_height, uint32_t dst_width, uint32_t dst_height,
                                              uint32_t channels, uint32_t batch_size, const void* src,
                                              uint32_t src_w_off, uint32_t src_h_off, void* dst, uint32_t dst_w_off,
                                              uint32_t dst_h_off, void* stream) {
  return slice2d(0, dtype, count_w, count_h, src_width, src_height, dst_width, dst_height, channels, batch_size, src,
                 src_w_off, src_h_off, dst, dst_w_off, dst_h_off, stream);
}

extern "C" int ad_slice2d_add_hw_nchw_packed(int32_t dtype, uint32_t count_w, uint32_t count_h, uint32_t src_width,
                                             uint32_t src_height, uint32_t dst_width, uint32_t dst_height,
                                             uint32_t channels, uint32_t batch_size, const void* src,
                                             uint32_t src_w_off, uint32_t src_h_off, void* dst, uint32_t dst_w_off,
                                             uint32_t dst_h_off, void* stream) {
  return slice2d(1, dtype, count_w, count_h, src_width, src_height, dst_width, dst_height, channels, batch_size, src,
                 src_w_off, src_h_off, dst, dst_w_off, dst_h_off, stream);
}


// ------------------------------------------------------------------------------------------ 2-D rank grids
namespace adk {
// Faces and corners of rank (gy, gx) in a grid_h x grid_w grid.  Every padded buffer holds (h + 2p) x (w + 2p)
// positions per plane with the interior at (p, p).  A region is (first row, row count, first column, column count)
// in padded coordinates.
struct Region { uint32_t y0, ny, x0, nx; };
// what rank r SENDS towards neighbour direction (dy, dx) -- its interior edge -- and where that lands in the
// neighbour's halo
static void halo2d_regions(int dy, int dx, uint32_t p, uint32_t w, uint32_t h, Region& mine, Region& theirs) {
  mine.y0 = dy < 0 ? p : dy > 0 ? h : p;           mine.ny = dy == 0 ? h : p;
  mine.x0 = dx < 0 ? p : dx > 0 ? w : p;           mine.nx = dx == 0 ? w : p;
  theirs.y0 = dy < 0 ? p + h : dy > 0 ? 0 : p;     theirs.ny = mine.ny;
  theirs.x0 = dx < 0 ? p + w : dx > 0 ? 0 : p;     theirs.nx = mine.nx;
}
static int check_halo2d(const ad_halo2d_args* a) {
  if (!a) return AD_ERR_BAD_ARG;
  if (elem_size(a->dtype) == 0) return AD_ERR_UNSUPPORTED;
  if (a->layout != AD_NCHW && a->layout != AD_NHWC) return AD_ERR_UNSUPPORTED;
  const uint32_t R = a->grid_w * a->grid_h;
  if (a->grid_w < 1 || a->grid_h < 1 || R > AD_MAX_PEERS) return AD_ERR_BAD_ARG;
  if (a->rank_count == 0 || a->rank_first + a->rank_count > R) return AD_ERR_BAD_ARG;
  if (a->base_width == 0 || a->base_height == 0 || a->num_channels == 0 || a->batch_size == 0) return AD_ERR_BAD_ARG;
  if (a->grid_h > 1 && a->base_height < 2 * a->halo_pad) return AD_ERR_BAD_ARG;
  if (a->grid_w > 1 && a->base_width < 2 * a->halo_pad) return AD_ERR_BAD_ARG;
  for (uint32_t r = 0; r < R; ++r) {
    if (!a->bufs[r]) return AD_ERR_BAD_ARG;
    if (((uintptr_t)a->bufs[r] % (uintptr_t)elem_size(a->dtype)) != 0) return AD_ERR_ALIGN;
  }
  return AD_OK;
}
// One launch per served rank and per phase: phase 0 = the two row faces, 1 = the two column faces, 2 = the corners.
// The exchange runs all phases in one launch (no two jobs write the same cells); the accumulate-back runs them one
// after another, because a corner cell of the interior receives a row face, a column face and a corner.
static int halo2d(const ad_halo2d_args* a, bool reduce, cudaStream_t stream) {
  int st = check_halo2d(a);
  if (st != AD_OK) return st;
  const uint32_t p = a->halo_pad, w = a->base_width, h = a->base_height, gw = a->grid_w, gh = a->grid_h;
  if (p == 0 || gw * gh == 1) return AD_OK;
  const unsigned long long es = (unsigned long long)elem_size(a->dtype);
  const unsigned long long Wp = w + 2ull * p, Hp = h + 2ull * p, C = a->num_channels, N = a->batch_size;
  const unsigned long long px = a->layout == AD_NCHW ? es : C * es;     // bytes of one pixel step along x
  bool want_signal = false;
  if (!reduce)
    for (uint32_t q = 0; q < gw * gh; ++q) want_signal |= (a->signal_flags[q] != nullptr);
  if (want_signal && !a->block_counter) return AD_ERR_BAD_ARG;
  for (uint32_t r = a->rank_first; r < a->rank_first + a->rank_count; ++r) {
    const int gy = (int)(r / gw), gx = (int)(r % gw);
    for (int phase = 0; phase < (reduce ? 3 : 1); ++phase) {
      SegParams prm{};
      prm.elem = (int)es;
      prm.accumulate = reduce ? 1 : 0;
      if (a->layout == AD_NCHW) { prm.planes = (uint32_t)(N * C); prm.src_plane_stride = Hp * Wp * es; prm.src_row_stride = Wp * es; }
      else { prm.planes = (uint32_t)N; prm.src_plane_stride = Hp * Wp * C * es; prm.src_row_stride = Wp * C * es; }
      prm.dst_plane_stride = prm.src_plane_stride;
      prm.dst_row_stride = prm.src_row_stride;
      int nj = 0;
      for (int dy = -1; dy <= 1; ++dy)
        for (int dx = -1; dx <= 1; ++dx) {
          if (!dy && !dx) continue;
          const int kind = (dy && dx) ? 2 : (dy ? 0 : 1);
          if (reduce && kind != phase) continue;
          const int ny = gy + dy, nx = gx + dx;
          if (ny < 0 || nx < 0 || ny >= (int)gh || nx >= (int)gw) continue;
          const uint32_t q = (uint32_t)ny * gw + (uint32_t)nx;
          Region mine, theirs;
          halo2d_regions(dy, dx, p, w, h, mine, theirs);
          SegJob jb{};
          if (!reduce && a->push) {            // my edge -> the neighbour's halo
            jb.src = (const char*)a->bufs[r]; jb.dst = (char*)a->bufs[q];
            jb.src_row0 = mine.y0; jb.dst_row0 = theirs.y0;
            jb.src_xoff = (uint32_t)(mine.x0 * px); jb.dst_xoff = (uint32_t)(theirs.x0 * px);
            jb.signal_rank = (int)q;
          } else if (!reduce) {                // pull: the neighbour's edge (towards me) -> my halo
            Region his, here;
            halo2d_regions(-dy, -dx, p, w, h, his, here);
            jb.src = (const char*)a->bufs[q]; jb.dst = (char*)a->bufs[r];
            jb.src_row0 = his.y0; jb.dst_row0 = here.y0;
            jb.src_xoff = (uint32_t)(his.x0 * px); jb.dst_xoff = (uint32_t)(here.x0 * px);
            jb.signal_rank = (int)r;
          } else {                             // accumulate-back: the neighbour's halo copy of my edge adds into my edge
            jb.src = (const char*)a->bufs[q]; jb.dst = (char*)a->bufs[r];
            jb.src_row0 = theirs.y0; jb.dst_row0 = mine.y0;
            jb.src_xoff = (uint32_t)(theirs.x0 * px); jb.dst_xoff = (uint32_t)(mine.x0 * px);
            jb.signal_rank = -1;
          }
          jb.rows = mine.ny;
          jb.seg_bytes = (uint32_t)(mine.nx * px);
          prm.jobs[nj++] = jb;
        }
      prm.njobs = nj;
      if (want_signal) {
        for (int j = 0; j < nj; ++j) {
          const int q = prm.jobs[j].signal_rank;
          if (q >= 0 && a->signal_flags[q]) { prm.signal_flags[q] = a->signal_flags[q]; prm.signal_mask |= 1u << q; }
        }
        prm.epoch = a->epoch;
        prm.epoch_base = (const unsigned long long*)a->epoch_base;
        prm.block_counter = a->block_counter;
      }
      st = launch_seg(prm, stream);
      if (st != AD_OK) return st;
    }
  }
  return AD_OK;
}
}  // namespace adk

extern "C" int ad_halo2d_exchange(const ad_halo2d_args* a, void* stream) { return adk::halo2d(a, false, as_stream(stream)); }
extern "C" int ad_halo2d_reduce(const ad_halo2d_args* a, void* stream) { return adk::halo2d(a, true, as_stream(stream)); }
