// Implicit-GEMM convolution on the 5th-generation tensor cores (tcgen05.mma, accumulators in
// tensor memory), operands staged by TMA tile loads into 128-byte-swizzled shared memory.
// NHWC bf16 activations, KRSC bf16 filters, fp32 accumulate.
//
//   forward / data gradient   conv_tc_fwd_kernel
//       GEMM  M = 128 output pixels (a TH x TW patch of one image), N = BN output channels,
//       K = taps x channels walked in 64-channel slabs.  For every (tap, slab) ONE 4-D TMA box
//       load fetches the shifted (dilated, strided) activation patch [128 pixels][64 ch], which
//       lands exactly in the K-major SWIZZLE_128B operand layout, so no im2col is materialised.
//       The data gradient of a stride-1 convolution is the same kernel run over dy with the
//       taps mirrored and the filter transposed to C,R,S,K.
//       Persistent CTAs (one per SM) loop over tiles; warp 0 = TMA producer, warp 1 = MMA
//       issuer (one elected thread), warps 2-5 = epilogue.  Two accumulators in tensor memory
//       let the epilogue of tile i overlap the MMAs of tile i+1.
//   filter gradient           conv_tc_wgrad_kernel
//       GEMM  M = 128 output channels of dy, N = BN input channels of x, K = pixels.  Both
//       operands are the NHWC tiles as TMA delivers them ([pixel][64 ch] rows), consumed as
//       MN-major operands.  The pixel range is split across CTAs; each split writes an fp32
//       partial to caller scratch and a second kernel sums the partials in a fixed order
//       (reproducible, no atomics).
//
// Every mbarrier wait is bounded; on expiry the kernel raises an abort flag, all roles leave
// their loops, tensor memory is freed and AD_ERR_TIMEOUT is written to a status word.
// No TMA load here uses cluster multicast.
#include "common.cuh"
#include <algorithm>

#include "tc_common.cuh"

#include <cstdlib>
#include <mutex>

namespace adk {
namespace tc {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    else
      cudaGetLastError();
  });
  return fn;
}

int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                   const uint32_t* box, const uint32_t* elem_strides) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return AD_ERR_CUDA;
  if (((uintptr_t)base & 15u) != 0) return AD_ERR_ALIGN;
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = elem_strides[i];
    if (box[i] == 0 || box[i] > 256) return AD_ERR_UNSUPPORTED;
  }
  for (int i = 1; i < rank; ++i) {
    gstr[i - 1] = strides_bytes[i];
    if (strides_bytes[i] % 16) return AD_ERR_ALIGN;
  }
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstr, bx, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? AD_OK : AD_ERR_CUDA;
}

constexpr int kTileM = 128;         // pixels (fwd) / dy channels (wgrad) per tile = TMEM lanes
constexpr int kSlabBytes = 16384;   // one [128 rows][64 bf16] swizzled operand slab
constexpr int kThreads = 192;       // filter-gradient kernel: warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int kFwdThreads = 320;    // forward kernel: warp 0 TMA, warp 1 MMA, two groups of 4 epilogue warps

struct FwdParams {
  uint32_t NI, OP, OQ, OC;  // output: images, rows, cols, channels
  uint32_t CK;              // reduction channels per tap (multiple of 64)
  uint32_t kh, kw, sh, sw, dh, dw;
  int32_t offy, offx;       // input row = oy*sh + r*dh + offy
  uint32_t TH, TW, tiles_y, tiles_x, tiles_n;
  uint32_t TN, tiles_b;     // a tile spans TN images of TH x TW pixels (small maps); tiles_b = ceil(NI / TN)
  long long out_pitch, out_plane;  // elements between output rows / images
  __nv_bfloat16* out;
  const float* bias;
  int32_t relu, accumulate;
  int32_t* status;
  int32_t tma_store;   // epilogue: stage 64-channel chunks in shared memory, one TMA tile store each
};

constexpr int kStagingBytes = 2 * 16384;

struct SmemCtl {
  unsigned long long full[8], empty[8], tfull[2], tempty[2], stg_full[2], stg_free[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ uint32_t pow2_cols(uint32_t c) {
  uint32_t p = 32;
  while (p < c) p <<= 1;
  return p;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(kFwdThreads, 1)
conv_tc_fwd_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_o, const FwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t kStageBytes = kSlabBytes + BN * 128;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* osm = smem + (size_t)STAGES * kStageBytes;
  SmemCtl* ctl = (SmemCtl*)(osm + kStagingBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t tiles_m = p.tiles_b * p.tiles_y * p.tiles_x;
  const uint32_t total_tiles = tiles_m * p.tiles_n;
  const uint32_t slabs = p.CK / 64;
  const uint32_t kiters = p.kh * p.kw * slabs;
  constexpr uint32_t kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // BN in {32,64,128,256} -> power of two

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&ctl->tfull[a]), 1);
      // an accumulator is drained by both epilogue groups when a tile has several 64-channel chunks
      mbar_init(smem_u32(&ctl->tempty[a]), (p.tma_store && BN >= 128) ? 8 : 4);
      mbar_init(smem_u32(&ctl->stg_full[a]), 4);
      mbar_init(smem_u32(&ctl->stg_free[a]), 1);
    }
    ctl->abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (p.tma_store) tma_prefetch_desc(&map_o);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abortf = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abortf; tile += gridDim.x) {
        const uint32_t tn = tile / tiles_m, tm = tile % tiles_m;
        const uint32_t tx = tm % p.tiles_x, ty = (tm / p.tiles_x) % p.tiles_y, n = tm / (p.tiles_x * p.tiles_y) * p.TN;
        const int x0 = (int)(tx * p.TW * p.sw) + p.offx, y0 = (int)(ty * p.TH * p.sh) + p.offy;
        bool ok = true;
        for (uint32_t r = 0; r < p.kh && ok; ++r)
          for (uint32_t s = 0; s < p.kw && ok; ++s)
            for (uint32_t cb = 0; cb < slabs; ++cb) {
              if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abortf)) { ok = false; break; }
              const uint32_t full = smem_u32(&ctl->full[stage]);
              uint8_t* st = smem + (size_t)stage * kStageBytes;
              mbar_expect_tx(full, kStageBytes);
              tma_load_4d(smem_u32(st), &map_a, full, (int)(cb * 64), x0 + (int)(s * p.dw), y0 + (int)(r * p.dh), (int)n);
              tma_load_2d(smem_u32(st + kSlabBytes), &map_b, full, (int)((r * p.kw + s) * p.CK + cb * 64), (int)(tn * BN));
              if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BN, 0, 0);
      uint32_t stage = 0, phase = 0, it = 0;
      for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abortf; tile += gridDim.x, ++it) {
        const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(smem_u32(&ctl->tempty[acc]), acc_phase ^ 1u, abortf)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        bool ok = true;
        for (uint32_t k = 0; k < kiters; ++k) {
          if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abortf)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
          const uint64_t da = smem_desc_sw128(sa, 16, 1024), db = smem_desc_sw128(sa + kSlabBytes, 16, 1024);
#pragma unroll
          for (uint32_t kk = 0; kk < 4; ++kk)  // 4 x (K = 16 bf16 = 32 bytes) inside the 128-byte row
            umma_bf16(d, da + 2 * kk, db + 2 * kk, idesc, (k | kk) != 0u);
          umma_commit(smem_u32(&ctl->empty[stage]));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(smem_u32(&ctl->tfull[acc]));
      }
    }
  } else {
    const uint32_t q = (uint32_t)warp & 3u;  // TMEM lane quarter this warp may read
    const uint32_t grp = ((uint32_t)warp - 2u) >> 2;   // epilogue warps 2..5 = group 0, 6..9 = group 1
    const bool leader = (((uint32_t)warp - 2u) & 3u) == 0u;
    uint32_t it = 0, gk = 0;   // gk: chunks this group has staged so far
    for (uint32_t tile = blockIdx.x; tile < total_tiles && !*abortf; tile += gridDim.x, ++it) {
      const uint32_t acc = it & 1u, acc_phase = (it >> 1) & 1u;
      const uint32_t tn = tile / tiles_m, tm = tile % tiles_m;
      const uint32_t tx = tm % p.tiles_x, ty = (tm / p.tiles_x) % p.tiles_y, n = tm / (p.tiles_x * p.tiles_y) * p.TN;
      const uint32_t m = q * 32 + lane;
      if (BN >= 64 && p.tma_store) {
        // 64-channel chunks of the tile go through a swizzled [128 px][64 ch] staging buffer and one TMA
        // tile store each: coalesced, clipped to the tensor, no per-thread scattered 16-byte stores.  The
        // two warp groups take alternate chunks (alternate tiles when a tile is one chunk), each with its
        // own staging buffer, so one group converts while the other group's store drains.
        constexpr uint32_t kChunks = BN / 64;
        if (kChunks == 1 && (it & 1u) != grp) continue;
        if (!mbar_wait(smem_u32(&ctl->tfull[acc]), acc_phase, abortf)) break;
        tc_fence_after();
        uint8_t* stg = osm + (size_t)grp * 16384;
        uint8_t* srow = stg + m * 128u;
        const uint32_t m7 = m & 7u;
        bool live = true;
#pragma unroll 1
        for (uint32_t c64 = (kChunks == 1 ? 0u : grp); c64 < kChunks && live; c64 += 2, ++gk) {
          uint32_t v[64];
          const uint32_t taddr = tmem_base + ((q * 32u) << 16) + acc * BN + c64 * 64;
          tmem_ld32(taddr, *(uint32_t(*)[32])&v[0]);
          tmem_ld32(taddr + 32, *(uint32_t(*)[32])&v[32]);
          tmem_ld_wait();
          if (c64 + 2 >= kChunks) {   // this warp's last read of the accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ctl->tempty[acc]));
          }
          bool ok = true;
          if (gk >= 1) ok = mbar_wait(smem_u32(&ctl->stg_free[grp]), (gk - 1u) & 1u, abortf);
          if (!__all_sync(0xffffffffu, ok)) { live = false; break; }
          const uint32_t cbase = tn * BN + c64 * 64;
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 64; ++j)
              if (cbase + j < p.OC) v[j] = __float_as_uint(__uint_as_float(v[j]) + p.bias[cbase + j]);
          }
          if (p.relu) {
#pragma unroll
            for (int j = 0; j < 64; ++j) v[j] = __float_as_uint(fmaxf(__uint_as_float(v[j]), 0.f));
          }
#pragma unroll
          for (uint32_t g8 = 0; g8 < 8; ++g8) {
            uint4 pk;
            __nv_bfloat162* p2 = (__nv_bfloat162*)&pk;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              p2[j] = __floats2bfloat162_rn(__uint_as_float(v[g8 * 8 + 2 * j]), __uint_as_float(v[g8 * 8 + 2 * j + 1]));
            *(uint4*)(srow + ((g8 ^ m7) * 16u)) = pk;
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&ctl->stg_full[grp]));
          if (leader && lane == 0) {
            if (mbar_wait(smem_u32(&ctl->stg_full[grp]), gk & 1u, abortf)) {
              if (cbase < p.OC)
                asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(&map_o),
                             "r"(smem_u32(stg)), "r"((int)cbase), "r"((int)(tx * p.TW)), "r"((int)(ty * p.TH)), "r"((int)n)
                             : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
              asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
              mbar_arrive(smem_u32(&ctl->stg_free[grp]));
            }
          }
          __syncwarp();
        }
        if (!live) break;
        continue;
      }
      if (grp != 0) continue;   // the scattered-store form is served by the first group alone
      if (!mbar_wait(smem_u32(&ctl->tfull[acc]), acc_phase, abortf)) break;
      tc_fence_after();
      const uint32_t mi = m / (p.TW * p.TH), mr = m - mi * (p.TW * p.TH);   // image inside the tile, pixel inside the image
      const uint32_t oy = ty * p.TH + mr / p.TW, ox = tx * p.TW + mr % p.TW, on = n + mi;
      const bool valid = oy < p.OP && ox < p.OQ && on < p.NI;
      __nv_bfloat16* orow = p.out + (long long)on * p.out_plane + (long long)oy * p.out_pitch + (long long)ox * p.OC;
#pragma unroll 1
      for (uint32_t ch = 0; ch < BN / 32; ++ch) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((q * 32u) << 16) + acc * BN + ch * 32, v);
        tmem_ld_wait();
        const uint32_t c0 = tn * BN + ch * 32;
        if (valid && c0 < p.OC) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t cg = c0 + g * 8;
            float f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              f[j] = __uint_as_float(v[g * 8 + j]);
              if (p.bias && cg + j < p.OC) f[j] += p.bias[cg + j];
            }
            if (cg + 8 <= p.OC && (p.OC & 7u) == 0) {
              if (p.accumulate) {
                uint4 old = *(const uint4*)(orow + cg);
                const __nv_bfloat162* o2 = (const __nv_bfloat162*)&old;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float2 t = __bfloat1622float2(o2[j]);
                  f[2 * j] += t.x; f[2 * j + 1] += t.y;
                }
              }
              if (p.relu) {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = fmaxf(f[j], 0.f);
              }
              uint4 pk;
              __nv_bfloat162* p2 = (__nv_bfloat162*)&pk;
#pragma unroll
              for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(f[2 * j], f[2 * j + 1]);
              *(uint4*)(orow + cg) = pk;
            } else {
              for (int j = 0; j < 8; ++j)
                if (cg + j < p.OC) {
                  float t = f[j];
                  if (p.accumulate) t += __bfloat162float(orow[cg + j]);
                  if (p.relu) t = fmaxf(t, 0.f);
                  orow[cg + j] = __float2bfloat16_rn(t);
                }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->tempty[acc]));
    }
    if (p.tma_store && leader && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  tc_fence_before();
  __syncthreads();
  if (*abortf) {
    // Let any tile copy that is still in flight land before shared memory is released.
    for (int i = 0; i < 2000; ++i) __nanosleep(500);
    if (threadIdx.x == 0 && p.status) *p.status = AD_ERR_TIMEOUT;
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------- filter gradient
struct WgParams {
  uint32_t NI, OP, OQ;  // dy: images, rows, cols
  uint32_t KO, CI;      // dy channels (GEMM M), x channels (GEMM N)
  uint32_t kh, kw, sh, sw, dh, dw;
  int32_t offy, offx;
  uint32_t TH, TW, tiles_y, tiles_x;
  uint32_t TN, tiles_b;  // a tile spans TN images (small maps); tiles_b = ceil(NI / TN)
  uint32_t ktiles, ctiles, splits;
  float* partial;       // [splits][KO][kh*kw][CI]
  int32_t* status;
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(kThreads, 1)
conv_tc_wgrad_kernel(const __grid_constant__ CUtensorMap map_dy, const __grid_constant__ CUtensorMap map_x,
                     const WgParams p) {
  extern __shared__ uint8_t smem_raw[];
  constexpr uint32_t kABytes = 2 * kSlabBytes, kBBytes = (BN / 64) * kSlabBytes, kStageBytes = kABytes + kBBytes;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  SmemCtl* ctl = (SmemCtl*)(smem + (size_t)STAGES * kStageBytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;

  // blockIdx.y -> (tap, k tile, c tile); blockIdx.x -> split of the pixel tiles
  const uint32_t split = blockIdx.x;
  uint32_t rem = blockIdx.y;
  const uint32_t ct = rem % p.ctiles; rem /= p.ctiles;
  const uint32_t kt = rem % p.ktiles; rem /= p.ktiles;
  const uint32_t tap = rem, r = tap / p.kw, s = tap % p.kw;
  const uint32_t sp_tiles = p.tiles_b * p.tiles_y * p.tiles_x;
  const uint32_t my_tiles = split < sp_tiles ? (sp_tiles - split + p.splits - 1) / p.splits : 0;

  if (threadIdx.x == 0) {
    for (int st = 0; st < STAGES; ++st) {
      mbar_init(smem_u32(&ctl->full[st]), 1);
      mbar_init(smem_u32(&ctl->empty[st]), 1);
    }
    mbar_init(smem_u32(&ctl->tfull[0]), 1);
    ctl->abort_flag = 0;
    mbar_init_fence();
    tma_prefetch_desc(&map_dy);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  volatile int* abortf = &ctl->abort_flag;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      for (uint32_t j = 0; j < my_tiles; ++j) {
        const uint32_t tm = split + j * p.splits;
        const uint32_t tx = tm % p.tiles_x, ty = (tm / p.tiles_x) % p.tiles_y, n = tm / (p.tiles_x * p.tiles_y) * p.TN;
        if (!mbar_wait(smem_u32(&ctl->empty[stage]), phase ^ 1u, abortf)) break;
        const uint32_t full = smem_u32(&ctl->full[stage]);
        uint8_t* st = smem + (size_t)stage * kStageBytes;
        mbar_expect_tx(full, kStageBytes);
        const int qx = (int)(tx * p.TW), qy = (int)(ty * p.TH);
        tma_load_4d(smem_u32(st), &map_dy, full, (int)(kt * 128), qx, qy, (int)n);
        tma_load_4d(smem_u32(st + kSlabBytes), &map_dy, full, (int)(kt * 128 + 64), qx, qy, (int)n);
        const int ix = qx * (int)p.sw + (int)(s * p.dw) + p.offx, iy = qy * (int)p.sh + (int)(r * p.dh) + p.offy;
#pragma unroll
        for (int b = 0; b < BN / 64; ++b)
          tma_load_4d(smem_u32(st + kABytes + b * kSlabBytes), &map_x, full, (int)(ct * BN + b * 64), ix, iy, (int)n);
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BN, 1, 1);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (uint32_t j = 0; j < my_tiles; ++j) {
        if (!mbar_wait(smem_u32(&ctl->full[stage]), phase, abortf)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)stage * kStageBytes);
#pragma unroll
        for (uint32_t ks = 0; ks < 8; ++ks) {  // 8 x (K = 16 pixels = 16 rows of 128 B)
          const uint64_t da = smem_desc_sw128(sa + ks * 2048, kSlabBytes, 1024);
          const uint64_t db = smem_desc_sw128(sa + kABytes + ks * 2048, kSlabBytes, 1024);
          umma_bf16(tmem_base, da, db, idesc, (j | ks) != 0u);
        }
        umma_commit(smem_u32(&ctl->empty[stage]));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (ok) umma_commit(smem_u32(&ctl->tfull[0]));
    }
  } else {
    const uint32_t q = (uint32_t)warp & 3u;
    const uint32_t taps = p.kh * p.kw;
    const uint32_t k = kt * 128 + q * 32 + lane;
    float* orow = p.partial + (((size_t)split * p.KO + k) * taps + tap) * p.CI + (size_t)ct * BN;
    if (my_tiles == 0) {
      if (k < p.KO)
        for (uint32_t c = 0; c < BN && ct * BN + c < p.CI; ++c) orow[c] = 0.f;
    } else if (mbar_wait(smem_u32(&ctl->tfull[0]), 0, abortf)) {
      tc_fence_after();
#pragma unroll 1
      for (uint32_t ch = 0; ch < BN / 32; ++ch) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((q * 32u) << 16) + ch * 32, v);
        tmem_ld_wait();
        if (k < p.KO) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const uint32_t c = ct * BN + ch * 32 + g * 4;
            if (c + 4 <= p.CI)
              *(float4*)(orow + ch * 32 + g * 4) = make_float4(__uint_as_float(v[g * 4]), __uint_as_float(v[g * 4 + 1]),
                                                               __uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3]));
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abortf) {
    for (int i = 0; i < 2000; ++i) __nanosleep(500);
    if (threadIdx.x == 0 && p.status) *p.status = AD_ERR_TIMEOUT;
  }
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// dw[i] (+)= sum over splits of partial[s][i], fixed order.
// taps, C: filter geometry; kcrs != 0 stores element (k, tap, c) at (k*C + c)*taps + tap instead of index i
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(size_t n, size_t part_stride, uint32_t splits,
                                                           const float* __restrict__ partial, float* dw, int accumulate,
                                                           uint32_t taps, uint32_t C, int kcrs) {
  // 64 outputs x 4 split lanes per block: lane l sums splits l, l+4, ... (8 loads in flight), lanes combine in order
  const uint32_t tx = threadIdx.x & 63, pl = threadIdx.x >> 6;
  const size_t i = (size_t)blockIdx.x * 64 + tx;
  float t = 0.f;
  if (i < n)
    for (uint32_t s0 = pl; s0 < splits; s0 += 32) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { const uint32_t si = s0 + 4 * u; v[u] = si < splits ? partial[(size_t)si * part_stride + i] : 0.f; }
#pragma unroll
      for (int u = 0; u < 8; ++u) t += v[u];
    }
  __shared__ float sh[4][64];
  sh[pl][tx] = t;
  __syncthreads();
  if (pl != 0 || i >= n) return;
  t = ((sh[0][tx] + sh[1][tx]) + sh[2][tx]) + sh[3][tx];
  size_t o = i;
  if (kcrs) {
    const uint32_t c = (uint32_t)(i % C);
    const size_t r = i / C;
    const uint32_t tap = (uint32_t)(r % taps);
    o = ((r / taps) * C + c) * taps + tap;
  }
  dw[o] = accumulate ? dw[o] + t : t;
}

// up[n][y][x][:] = dy[n][y/sh][x/sw][:] where both divisions are exact, else 0  (16-byte groups of channels)
__global__ void __launch_bounds__(256) zero_insert_kernel(const uint4* __restrict__ dy, uint4* up, uint32_t N, uint32_t P,
                                                          uint32_t Q, uint32_t DP, uint32_t DQ, uint32_t G, uint32_t sh,
                                                          uint32_t sw) {
  const size_t total = (size_t)N * DP * DQ * G, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t g = (uint32_t)(i % G);
    size_t r = i / G;
    const uint32_t x = (uint32_t)(r % DQ); r /= DQ;
    const uint32_t y = (uint32_t)(r % DP), n = (uint32_t)(r / DP);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (y % sh == 0 && x % sw == 0) v = dy[(((size_t)n * P + y / sh) * Q + x / sw) * G + g];
    up[i] = v;
  }
}

// Filter for the data gradient: wt[c][kh-1-r][kw-1-s][k] = w[k][r][s][c]  (bf16); rows of Kp >= K
// entries, zero past K.
__global__ void __launch_bounds__(256) filter_transpose_flip_kernel(uint32_t K, uint32_t Kp, uint32_t kh, uint32_t kw,
                                                                    uint32_t C, const __nv_bfloat16* __restrict__ w,
                                                                    __nv_bfloat16* wt) {
  const size_t total = (size_t)Kp * kh * kw * C, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    uint32_t k = (uint32_t)(i % Kp);
    size_t rr = i / Kp;
    uint32_t s = (uint32_t)(rr % kw); rr /= kw;
    uint32_t r = (uint32_t)(rr % kh);
    uint32_t c = (uint32_t)(rr / kh);
    wt[i] = k < K ? w[(((size_t)k * kh + (kh - 1 - r)) * kw + (kw - 1 - s)) * C + c] : __float2bfloat16_rn(0.f);
  }
}
// dst[pixel][0..Kp) = src[pixel][0..K), zero past K
__global__ void __launch_bounds__(256) pad_channels_kernel(size_t pixels, uint32_t K, uint32_t Kp,
                                                           const __nv_bfloat16* __restrict__ src, __nv_bfloat16* dst) {
  const size_t total = pixels * Kp, nt = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += nt) {
    const uint32_t k = (uint32_t)(i % Kp);
    const size_t px = i / Kp;
    dst[i] = k < K ? src[px * K + k] : __float2bfloat16_rn(0.f);
  }
}

// db[k] (+)= sum over pixels of dy[pixel][k] (dense NHWC bf16), in two fixed-order stages: block (channel group,
// split) sums its share of the pixels into part[split][k], bias_grad_finish adds the splits in order.
__global__ void __launch_bounds__(256) bias_grad_nhwc_kernel(size_t pixels, uint32_t K, const __nv_bfloat16* __restrict__ dy,
                                                             float* part) {
  const uint32_t k = blockIdx.x * 32 + threadIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const size_t chunk = (pixels + nsplit - 1) / nsplit, lo = (size_t)split * chunk, hi = lo + chunk < pixels ? lo + chunk : pixels;
  float acc = 0.f;
  if (k < K)
    for (size_t i = lo + threadIdx.y; i < hi; i += 8) acc += __bfloat162float(dy[i * K + k]);
  __shared__ float red[8][33];
  red[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && k < K) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    part[(size_t)split * K + k] = t;
  }
}
__global__ void bias_grad_finish(uint32_t K, uint32_t nsplit, const float* __restrict__ part, float* db, int accumulate) {
  const uint32_t k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  float t = 0.f;
  for (uint32_t s = 0; s < nsplit; ++s) t += part[(size_t)s * K + k];
  db[k] = accumulate ? db[k] + t : t;
}
// `part`: scratch of at least 64 * K floats (the filter-gradient partials, free again once they are reduced)
static void launch_bias_grad(size_t pixels, uint32_t K, const void* dy, float* db, int accumulate, float* part, cudaStream_t s) {
  const uint32_t nsplit = (uint32_t)std::min<size_t>(64, std::max<size_t>(1, pixels / 512));
  dim3 grid((K + 31) / 32, nsplit), block(32, 8);
  bias_grad_nhwc_kernel<<<grid, block, 0, s>>>(pixels, K, (const __nv_bfloat16*)dy, part);
  bias_grad_finish<<<(K + 127) / 128, 128, 0, s>>>(K, nsplit, part, db, accumulate);
  count_launch(2);
}

// ---------------------------------------------------------------- host side
struct Geo {
  uint32_t P, Q;
};
static int conv_geo(const ad_conv2d_args* a, Geo& g) {
  if (!a) return AD_ERR_BAD_ARG;
  if (a->N == 0 || a->C == 0 || a->H == 0 || a->W == 0 || a->K == 0 || a->kh == 0 || a->kw == 0) return AD_ERR_BAD_ARG;
  if (a->stride_h == 0 || a->stride_w == 0 || a->dil_h == 0 || a->dil_w == 0) return AD_ERR_BAD_ARG;
  const long long eh = (long long)a->H + 2ll * a->pad_h - (long long)a->dil_h * (a->kh - 1) - 1;
  const long long ew = (long long)a->W + 2ll * a->pad_w - (long long)a->dil_w * (a->kw - 1) - 1;
  if (eh < 0 || ew < 0) return AD_ERR_BAD_ARG;
  g.P = (uint32_t)(eh / a->stride_h + 1);
  g.Q = (uint32_t)(ew / a->stride_w + 1);
  return AD_OK;
}

// Patch of 128 output pixels (TN images x TH rows x TW columns) wasting the fewest lanes on partial tiles: large
// maps get one image per tile, small feature maps (7 x 7, 14 x 14) several, which otherwise leave most of a
// 128-pixel tile empty.
static void pick_tile3(uint32_t NI, uint32_t OP, uint32_t OQ, uint32_t sh, uint32_t sw, uint32_t& TN, uint32_t& TH, uint32_t& TW) {
  unsigned long long best = ~0ull;
  TN = 1; TH = 1; TW = 128;
  for (uint32_t tn = 1; tn <= 16; tn <<= 1)
    for (uint32_t tw = 128 / tn; tw >= 8; tw >>= 1) {
      const uint32_t th = 128 / tn / tw;
      if (th == 0 || tw * sw > 256 || th * sh > 256) continue;
      const unsigned long long cost = (unsigned long long)((OQ + tw - 1) / tw * tw) * ((OP + th - 1) / th * th) * ((NI + tn - 1) / tn * tn);
      if (cost < best) { best = cost; TN = tn; TH = th; TW = tw; }
    }
}

template <int BN>
static int launch_fwd(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const FwdParams& p, cudaStream_t s) {
  constexpr int kStageBytes = kSlabBytes + BN * 128;
  constexpr int STAGES = (192 * 1024) / kStageBytes > 8 ? 8 : (192 * 1024) / kStageBytes;
  constexpr int smem = STAGES * kStageBytes + kStagingBytes + 1024 + (int)sizeof(SmemCtl);
  static unsigned attr_done = 0;  // one bit per device: the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_done & (1u << (dev & 31)))) {
    if (cudaFuncSetAttribute(conv_tc_fwd_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess) {
      cudaGetLastError();
      return AD_ERR_CUDA;
    }
    attr_done |= 1u << (dev & 31);
  }
  const uint32_t total = p.tiles_b * p.tiles_y * p.tiles_x * p.tiles_n;
  const unsigned grid = total < (uint32_t)kNumSMs ? total : kNumSMs;
  conv_tc_fwd_kernel<BN, STAGES><<<grid, kFwdThreads, smem, s>>>(ma, mb, mo, p);
  count_launch();
  return launch_status();
}

int conv_tc_row_fwd(const void* act, uint32_t NI, uint32_t IH, uint32_t IW, uint32_t CK, const void* filt, uint32_t OC,
                    uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw, int offy, int offx,
                    uint32_t OP, uint32_t OQ, void* out, long long out_pitch, long long out_plane, const float* bias,
                    int relu, int accumulate, int32_t* status, cudaStream_t s);

size_t conv_tc_row_wgrad_scratch(uint32_t NI, uint32_t CI, uint32_t KO, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw,
                                 uint32_t dh, uint32_t dw, uint32_t OP, uint32_t OQ);
int conv_tc_row_wgrad(const void* x, uint32_t NI, uint32_t IH, uint32_t IW, uint32_t CI, const void* dy, uint32_t KO,
                      uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw, int offy, int offx,
                      uint32_t OP, uint32_t OQ, float* dwt, int accumulate, int kcrs, void* partial, size_t partial_bytes,
                      int32_t* status, cudaStream_t s);

// Generic forward-style implicit GEMM launch (fprop, or dgrad expressed as fprop).
static int run_fwd_gemm(const void* act, uint32_t NI, uint32_t IH, uint32_t IW, uint32_t CK, const void* filt,
                        uint32_t OC, uint32_t kh, uint32_t kw, uint32_t sh, uint32_t sw, uint32_t dh, uint32_t dw,
                        int offy, int offx, uint32_t OP, uint32_t OQ, void* out, long long out_pitch,
                        long long out_plane, const float* bias, int relu, int accumulate, int32_t* status,
                        cudaStream_t s) {
  if (CK % 64 != 0) return AD_ERR_UNSUPPORTED;
  if (!getenv("ARRAYDIFF_B200_NO_ROW_KERNEL")) {
    // 64-channel layers: the row-tile kernel fetches each activation patch once (conv_tc_row.cu)
    int st = conv_tc_row_fwd(act, NI, IH, IW, CK, filt, OC, kh, kw, sh, sw, dh, dw, offy, offx, OP, OQ, out, out_pitch,
                             out_plane, bias, relu, accumulate, status, s);
    if (st != AD_ERR_UNSUPPORTED) {
      g_last_conv_kernel = kConvTcRow;
      return st;
    }
  }
  g_last_conv_kernel = kConvTcGeneral;
  FwdParams p{};
  p.NI = NI; p.OP = OP; p.OQ = OQ; p.OC = OC; p.CK = CK;
  p.kh = kh; p.kw = kw; p.sh = sh; p.sw = sw; p.dh = dh; p.dw = dw; p.offy = offy; p.offx = offx;
  pick_tile3(NI, OP, OQ, sh, sw, p.TN, p.TH, p.TW);
  p.tiles_y = (OP + p.TH - 1) / p.TH;
  p.tiles_x = (OQ + p.TW - 1) / p.TW;
  p.tiles_b = (NI + p.TN - 1) / p.TN;
  const int BN = OC > 128 ? 256 : (OC > 64 ? 128 : (OC > 32 ? 64 : 32));
  p.tiles_n = (OC + BN - 1) / BN;
  p.out_pitch = out_pitch ? out_pitch : (long long)OQ * OC;
  p.out_plane = out_plane ? out_plane : (long long)OP * OQ * OC;
  if (((uintptr_t)out & 15u) || (p.out_pitch % 8) || (p.out_plane % 8)) {
    if ((OC & 7u) == 0) return AD_ERR_ALIGN;
  }
  p.out = (__nv_bfloat16*)out;
  p.bias = bias; p.relu = relu; p.accumulate = accumulate; p.status = status;

  CUtensorMap ma, mb;
  {
    uint64_t dims[4] = {CK, IW, IH, NI};
    uint64_t str[4] = {0, (uint64_t)CK * 2, (uint64_t)IW * CK * 2, (uint64_t)IH * IW * CK * 2};
    uint32_t box[4] = {64, p.TW * sw, p.TH * sh, p.TN};
    uint32_t es[4] = {1, sw, sh, 1};
    int st = make_tmap_bf16(&ma, act, 4, dims, str, box, es);
    if (st != AD_OK) return st;
  }
  {
    uint64_t dims[2] = {(uint64_t)kh * kw * CK, OC};
    uint64_t str[2] = {0, (uint64_t)kh * kw * CK * 2};
    uint32_t box[2] = {64, (uint32_t)BN};
    uint32_t es[2] = {1, 1};
    int st = make_tmap_bf16(&mb, filt, 2, dims, str, box, es);
    if (st != AD_OK) return st;
  }
  CUtensorMap mo = ma;
  p.tma_store = (!accumulate && BN >= 64 && (OC & 7u) == 0 && !((uintptr_t)out & 15u) && (p.out_pitch % 8) == 0 &&
                 (p.out_plane % 8) == 0) ? 1 : 0;
  if (p.tma_store) {
    uint64_t dims[4] = {OC, OQ, OP, NI};
    uint64_t str[4] = {0, (uint64_t)OC * 2, (uint64_t)p.out_pitch * 2, (uint64_t)p.out_plane * 2};
    uint32_t box[4] = {64, p.TW, p.TH, p.TN};
    uint32_t es[4] = {1, 1, 1, 1};
    int st = make_tmap_bf16(&mo, out, 4, dims, str, box, es);
    if (st != AD_OK) return st;
  }
  switch (BN) {
    case 256: return launch_fwd<256>(ma, mb, mo, p, s);
    case 128: return launch_fwd<128>(ma, mb, mo, p, s);
    case 64: return launch_fwd<64>(ma, mb, mo, p, s);
    default: return launch_fwd<32>(ma, mb, mo, p, s);
  }
}

template <int BN>
static int launch_wgrad(const CUtensorMap& mdy, const CUtensorMap& mx, const WgParams& p, cudaStream_t s) {
  constexpr int kStageBytes = 2 * kSlabBytes + (BN / 64) * kSlabBytes;
  constexpr int STAGES = (200 * 1024) / kStageBytes;
  constexpr int smem = STAGES * kStageBytes + 1024 + (int)sizeof(SmemCtl);
  static unsigned attr_done = 0;  // one bit per device: the attribute is per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (!(attr_done & (1u << (dev & 31)))) {
    if (cudaFuncSetAttribute(conv_tc_wgrad_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
        cudaSuccess) {
      cudaGetLastError();
      return AD_ERR_CUDA;
    }
    attr_done |= 1u << (dev & 31);
  }
  dim3 grid(p.splits, p.kh * p.kw * p.ktiles * p.ctiles);
  conv_tc_wgrad_kernel<BN, STAGES><<<grid, kThreads, smem, s>>>(mdy, mx, p);
  count_launch();
  return launch_status();
}

// Input channels per CTA of the general filter-gradient kernel.  (A 256-wide tile halves the L2 fetches of the dy
// tile but leaves room for two pipeline stages only: measured 15 % slower on the 512 -> 512 layers.)
static int wgrad_bn(uint32_t C) { return C > 64 ? 128 : 64; }

static uint32_t wgrad_splits(uint32_t sp_tiles, uint32_t outer) {
  uint32_t want = (2 * kNumSMs + outer - 1) / outer;
  if (want > sp_tiles) want = sp_tiles;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return want;
}

static size_t round_1k(size_t b) { return (b + 1023) / 1024 * 1024; }
// Gradient channel counts the tensor-core kernels take as they are: the data gradient reduces over K in
// 64-channel slabs, the filter gradient needs 16-byte pixel pitches of dy.  Other counts (a 19-class head)
// run on a zero-padded copy of dy kept in scratch.
static uint32_t dgrad_kp(uint32_t K) { return (K + 63) / 64 * 64; }
static uint32_t wgrad_kp(uint32_t K) { return (K + 7) / 8 * 8; }

// Scratch layouts:
//   pass 1 (data gradient):   [status 16 B | transposed filter C,R,S,Kp bf16] [dy padded to Kp channels, if Kp != K]
//                             [dy with zeros inserted, if strided]
//   pass 2 (filter gradient): [status 16 B] [dy padded, if Kp != K] [fp32 partials]
size_t conv_tc_scratch_bytes(const ad_conv2d_args* a, int pass) {
  Geo g;
  if (conv_geo(a, g) != AD_OK) return 0;
  const size_t pixels = (size_t)a->N * g.P * g.Q;
  if (pass == 1) {
    const uint32_t Kp = dgrad_kp(a->K);
    size_t b = round_1k((size_t)Kp * a->kh * a->kw * a->C * 2 + 16);
    if (Kp != a->K) b += round_1k(pixels * Kp * 2);
    if (a->stride_h != 1 || a->stride_w != 1)
      b += round_1k((size_t)a->N * ((g.P - 1) * a->stride_h + 1) * ((g.Q - 1) * a->stride_w + 1) * Kp * 2);
    return b;
  }
  if (pass == 2) {
    const uint32_t Kp = wgrad_kp(a->K);
    const size_t wcount = (size_t)Kp * a->kh * a->kw * a->C;
    uint32_t TN, TH, TW;
    pick_tile3(a->N, g.P, g.Q, a->stride_h, a->stride_w, TN, TH, TW);
    const uint32_t sp = ((a->N + TN - 1) / TN) * ((g.P + TH - 1) / TH) * ((g.Q + TW - 1) / TW);
    const uint32_t BN = (uint32_t)wgrad_bn(a->C);
    const uint32_t outer = a->kh * a->kw * ((Kp + 127) / 128) * ((a->C + BN - 1) / BN);
    size_t general = (size_t)wgrad_splits(sp, outer) * wcount * 4;
    size_t row = conv_tc_row_wgrad_scratch(a->N, a->C, a->K, a->kh, a->kw, a->stride_h, a->stride_w, a->dil_h, a->dil_w, g.P, g.Q);
    size_t b = 1024 + (general > row ? general : row);
    if (Kp != a->K) b += round_1k(pixels * Kp * 2);
    return b;
  }
  return 16;
}

int conv_tc_fprop(const ad_conv2d_args* a, cudaStream_t s) {
  Geo g;
  int st = conv_geo(a, g);
  if (st != AD_OK) return st;
  if (!a->x || !a->w || !a->y) return AD_ERR_BAD_ARG;
  if (a->pad_h || a->pad_w) {
    // Implicit padding is served by TMA's out-of-bounds zero fill (negative start coordinates).
  }
  int32_t* status = (a->scratch && a->scratch_bytes >= 16) ? (int32_t*)a->scratch : nullptr;
  // A row range is the same problem with fewer output rows: shift the input row offset and the
  // output pointer, keep the pitches of the full tensor.
  uint32_t q0 = 0, nq = g.P;
  if (a->out_row_count) {
    if ((unsigned long long)a->out_row_begin + a->out_row_count > g.P) return AD_ERR_BAD_ARG;
    q0 = a->out_row_begin; nq = a->out_row_count;
  }
  const long long pitch = a->y_pitch ? a->y_pitch : (long long)g.Q * a->K;
  const long long plane = a->y_plane ? a->y_plane : (long long)g.P * g.Q * a->K;
  __nv_bfloat16* out = (__nv_bfloat16*)a->y + (long long)q0 * pitch;
  return run_fwd_gemm(a->x, a->N, a->H, a->W, a->C, a->w, a->K, a->kh, a->kw, a->stride_h, a->stride_w, a->dil_h,
                      a->dil_w, -(int)a->pad_h + (int)(q0 * a->stride_h), -(int)a->pad_w, nq, g.Q, out, pitch, plane, a->bias,
                      a->relu, 0, status, s);
}

int conv_tc_dgrad(const ad_conv2d_args* a, cudaStream_t s) {
  Geo g;
  int st = conv_geo(a, g);
  if (st != AD_OK) return st;
  if (!a->y || !a->w || !a->dx || !a->scratch) return AD_ERR_BAD_ARG;
  if (a->y_pitch || a->y_plane) return AD_ERR_UNSUPPORTED;  // dy must be dense for the TMA view
  if (a->scratch_bytes < conv_tc_scratch_bytes(a, 1)) return AD_ERR_SCRATCH;
  const uint32_t Kp = dgrad_kp(a->K);
  int32_t* status = (int32_t*)a->scratch;
  __nv_bfloat16* wt = (__nv_bfloat16*)((char*)a->scratch + 16);
  char* next = (char*)a->scratch + round_1k((size_t)Kp * a->kh * a->kw * a->C * 2 + 16);
  const size_t wcount = (size_t)Kp * a->kh * a->kw * a->C;
  filter_transpose_flip_kernel<<<grid_for(wcount, 256), 256, 0, s>>>(a->K, Kp, a->kh, a->kw, a->C,
                                                                     (const __nv_bfloat16*)a->w, wt);
  count_launch();
  const void* dy = a->y;
  if (Kp != a->K) {
    const size_t pixels = (size_t)a->N * g.P * g.Q;
    pad_channels_kernel<<<grid_for(pixels * Kp, 256, 16), 256, 0, s>>>(pixels, a->K, Kp, (const __nv_bfloat16*)a->y,
                                                                        (__nv_bfloat16*)next);
    count_launch();
    dy = next;
    next += round_1k(pixels * Kp * 2);
  }
  // dx[n,yy,xx,c] = sum_{r',s',k} dy[n, yy + ph - (kh-1)*dh + r'*dh, xx + ..., k] * wt[c][r'][s'][k]
  const int offy = (int)a->pad_h - (int)((a->kh - 1) * a->dil_h), offx = (int)a->pad_w - (int)((a->kw - 1) * a->dil_w);
  uint32_t DP = g.P, DQ = g.Q;
  if (a->stride_h != 1 || a->stride_w != 1) {
    // Strided layer: the data gradient is the stride-1 gradient of dy with (stride - 1) zeros inserted
    // between its pixels.  The zero-inserted copy lives in scratch; the tensor-core kernel then runs
    // unchanged (and multiplies the zeros -- strided layers are few).
    DP = (g.P - 1) * a->stride_h + 1; DQ = (g.Q - 1) * a->stride_w + 1;
    const size_t total8 = (size_t)a->N * DP * DQ * (Kp / 8);
    zero_insert_kernel<<<grid_for(total8, 256, 16), 256, 0, s>>>((const uint4*)dy, (uint4*)next, a->N, g.P, g.Q, DP, DQ,
                                                                   Kp / 8, a->stride_h, a->stride_w);
    count_launch();
    dy = next;
  }
  // A column range is the same problem with fewer output columns: shift the input column offset and the
  // output pointer, keep the pitches of the full tensor.
  uint32_t c0 = 0, nc = a->W;
  if (a->dx_col_count) {
    if ((unsigned long long)a->dx_col_begin + a->dx_col_count > a->W) return AD_ERR_BAD_ARG;
    c0 = a->dx_col_begin; nc = a->dx_col_count;
  }
  return run_fwd_gemm(dy, a->N, DP, DQ, Kp, wt, a->C, a->kh, a->kw, 1, 1, a->dil_h, a->dil_w, offy, offx + (int)c0, a->H,
                      nc, (__nv_bfloat16*)a->dx + (size_t)c0 * a->C, (long long)a->W * a->C, (long long)a->H * a->W * a->C,
                      nullptr, 0, a->accumulate, status, s);
}

int conv_tc_wgrad(const ad_conv2d_args* a, cudaStream_t s) {
  Geo g;
  int st = conv_geo(a, g);
  if (st != AD_OK) return st;
  if (!a->x || !a->y || !a->dw || !a->scratch) return AD_ERR_BAD_ARG;
  if (a->y_pitch || a->y_plane) return AD_ERR_UNSUPPORTED;
  if (a->C % 64 != 0) return AD_ERR_UNSUPPORTED;
  if (a->scratch_bytes < conv_tc_scratch_bytes(a, 2)) return AD_ERR_SCRATCH;
  const uint32_t Kp = wgrad_kp(a->K);
  const void* dy = a->y;
  char* part_base = (char*)a->scratch + 1024;
  if (Kp != a->K) {
    const size_t pixels = (size_t)a->N * g.P * g.Q;
    pad_channels_kernel<<<grid_for(pixels * Kp, 256, 16), 256, 0, s>>>(pixels, a->K, Kp, (const __nv_bfloat16*)a->y,
                                                                        (__nv_bfloat16*)part_base);
    count_launch();
    dy = part_base;
    part_base += round_1k(pixels * Kp * 2);
  }
  const size_t part_bytes = a->scratch_bytes - (size_t)(part_base - (char*)a->scratch);
  if (Kp == a->K && !getenv("ARRAYDIFF_B200_NO_ROW_KERNEL")) {
    // 64-channel layers: one CTA serves all taps from one fetch of x and dy (conv_tc_row.cu)
    st = conv_tc_row_wgrad(a->x, a->N, a->H, a->W, a->C, a->y, a->K, a->kh, a->kw, a->stride_h, a->stride_w, a->dil_h,
                           a->dil_w, -(int)a->pad_h, -(int)a->pad_w, g.P, g.Q, (float*)a->dw, a->accumulate, a->dw_kcrs,
                           part_base, part_bytes, (int32_t*)a->scratch, s);
    if (st == AD_OK && a->db) launch_bias_grad((size_t)a->N * g.P * g.Q, a->K, a->y, a->db, a->accumulate, (float*)part_base, s);
    if (st != AD_ERR_UNSUPPORTED) {
      g_last_conv_kernel = kConvTcRow;
      return st;
    }
  }
  g_last_conv_kernel = kConvTcGeneral;
  WgParams p{};
  p.NI = a->N; p.OP = g.P; p.OQ = g.Q; p.KO = Kp; p.CI = a->C;
  p.kh = a->kh; p.kw = a->kw; p.sh = a->stride_h; p.sw = a->stride_w; p.dh = a->dil_h; p.dw = a->dil_w;
  p.offy = -(int)a->pad_h; p.offx = -(int)a->pad_w;
  // The tile is chosen for the dy grid; the x box is the same patch scaled by the stride.
  pick_tile3(a->N, g.P, g.Q, a->stride_h, a->stride_w, p.TN, p.TH, p.TW);
  p.tiles_y = (g.P + p.TH - 1) / p.TH;
  p.tiles_x = (g.Q + p.TW - 1) / p.TW;
  p.tiles_b = (a->N + p.TN - 1) / p.TN;
  const int BN = wgrad_bn(a->C);
  p.ktiles = (Kp + 127) / 128;
  p.ctiles = (a->C + BN - 1) / BN;
  const uint32_t sp_tiles = p.tiles_b * p.tiles_y * p.tiles_x;
  p.splits = wgrad_splits(sp_tiles, p.kh * p.kw * p.ktiles * p.ctiles);
  p.status = (int32_t*)a->scratch;
  p.partial = (float*)part_base;
  const size_t wcount = (size_t)a->K * a->kh * a->kw * a->C, wcount_p = (size_t)Kp * a->kh * a->kw * a->C;
  if (part_bytes < (size_t)p.splits * wcount_p * 4) return AD_ERR_SCRATCH;

  CUtensorMap mdy, mx;
  {
    uint64_t dims[4] = {Kp, g.Q, g.P, a->N};
    uint64_t str[4] = {0, (uint64_t)Kp * 2, (uint64_t)g.Q * Kp * 2, (uint64_t)g.P * g.Q * Kp * 2};
    uint32_t box[4] = {64, p.TW, p.TH, p.TN};
    uint32_t es[4] = {1, 1, 1, 1};
    st = make_tmap_bf16(&mdy, dy, 4, dims, str, box, es);
    if (st != AD_OK) return st;
  }
  {
    uint64_t dims[4] = {a->C, a->W, a->H, a->N};
    uint64_t str[4] = {0, (uint64_t)a->C * 2, (uint64_t)a->W * a->C * 2, (uint64_t)a->H * a->W * a->C * 2};
    uint32_t box[4] = {64, p.TW * a->stride_w, p.TH * a->stride_h, p.TN};
    uint32_t es[4] = {1, a->stride_w, a->stride_h, 1};
    st = make_tmap_bf16(&mx, a->x, 4, dims, str, box, es);
    if (st != AD_OK) return st;
  }
  st = BN == 128 ? launch_wgrad<128>(mdy, mx, p, s) : launch_wgrad<64>(mdy, mx, p, s);
  if (st != AD_OK) return st;
  wgrad_reduce_kernel<<<(unsigned)((wcount + 63) / 64), 256, 0, s>>>(wcount, wcount_p, p.splits, p.partial, (float*)a->dw, a->accumulate,
                                                                      a->kh * a->kw, a->C, a->dw_kcrs);
  count_launch();
  if (a->db) launch_bias_grad((size_t)a->N * g.P * g.Q, a->K, a->y, a->db, a->accumulate, p.partial, s);
  return launch_status();
}

}  // namespace tc

// fp32 direct path (conv_direct.cu)
int conv_direct_fprop(const ad_conv2d_args* a, cudaStream_t s);
int conv_direct_dgrad(const ad_conv2d_args* a, cudaStream_t s);
int conv_direct_wgrad(const ad_conv2d_args* a, cudaStream_t s);

}  // namespace adk

using namespace adk;

static int path_of(const ad_conv2d_args* a) {
  if (!a) return -1;
  if (a->dtype == AD_F32 && a->layout == AD_NCHW) return 0;
  if (a->dtype == AD_BF16 && a->layout == AD_NHWC) return 1;
  return -1;
}

extern "C" size_t ad_conv2d_scratch_bytes(const ad_conv2d_args* a, int32_t pass) {
  if (path_of(a) != 1) return 0;
  return tc::conv_tc_scratch_bytes(a, pass);
}

// ---------------------------------------------------------------- per-call timing (ad_conv2d_profile)
#include <mutex>
#include <vector>
namespace {
struct ProfRec {
  ad_conv2d_profile_entry e;
  cudaEvent_t e0, e1;
};
std::mutex g_prof_mu;
bool g_prof_on = false;
std::vector<ProfRec> g_prof;

template <typename F>
int profiled(int pass, const ad_conv2d_args* a, void* stream, F&& call) {
  if (!g_prof_on || !a) return call();
  ProfRec r{};
  if (cudaEventCreate(&r.e0) != cudaSuccess || cudaEventCreate(&r.e1) != cudaSuccess) {
    cudaGetLastError();
    return call();
  }
  cudaEventRecord(r.e0, as_stream(stream));
  const int st = call();
  cudaEventRecord(r.e1, as_stream(stream));
  r.e.pass = pass; r.e.kernel = g_last_conv_kernel; r.e.status = st;
  r.e.N = a->N; r.e.C = a->C; r.e.H = a->H; r.e.W = a->W; r.e.K = a->K; r.e.kh = a->kh; r.e.kw = a->kw;
  r.e.stride = a->stride_h; r.e.dil = a->dil_h; r.e.pad = a->pad_h;
  r.e.out_rows = pass == 0 ? a->out_row_count : 0;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_prof.push_back(r);
  return st;
}
}  // namespace

extern "C" int ad_conv2d_profile(int32_t enable) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  for (auto& r : g_prof) { cudaEventDestroy(r.e0); cudaEventDestroy(r.e1); }
  g_prof.clear();
  g_prof_on = enable != 0;
  return AD_OK;
}
extern "C" size_t ad_conv2d_profile_read(ad_conv2d_profile_entry* out, size_t max_entries) {
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (!out) return g_prof.size();
  size_t n = 0;
  for (auto& r : g_prof) {
    if (n == max_entries) break;
    cudaEventSynchronize(r.e1);
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) { cudaGetLastError(); ms = -1.f; }
    r.e.ms = ms;
    out[n++] = r.e;
  }
  return n;
}

extern "C" int ad_conv2d_fprop(const ad_conv2d_args* a, void* stream) {
  return profiled(0, a, stream, [&] {
    switch (path_of(a)) {
      case 0: g_last_conv_kernel = kConvDirectF32; return conv_direct_fprop(a, as_stream(stream));
      case 1: return tc::conv_tc_fprop(a, as_stream(stream));
      default: return (int)(a ? AD_ERR_UNSUPPORTED : AD_ERR_BAD_ARG);
    }
  });
}
extern "C" int ad_conv2d_dgrad(const ad_conv2d_args* a, void* stream) {
  return profiled(1, a, stream, [&] {
    switch (path_of(a)) {
      case 0: g_last_conv_kernel = kConvDirectF32; return conv_direct_dgrad(a, as_stream(stream));
      case 1: return tc::conv_tc_dgrad(a, as_stream(stream));
      default: return (int)(a ? AD_ERR_UNSUPPORTED : AD_ERR_BAD_ARG);
    }
  });
}
extern "C" int ad_conv2d_wgrad(const ad_conv2d_args* a, void* stream) {
  return profiled(2, a, stream, [&] {
    switch (path_of(a)) {
      case 0: g_last_conv_kernel = kConvDirectF32; return conv_direct_wgrad(a, as_stream(stream));
      case 1: return tc::conv_tc_wgrad(a, as_stream(stream));
      default: return (int)(a ? AD_ERR_UNSUPPORTED : AD_ERR_BAD_ARG);
    }
  });
}
