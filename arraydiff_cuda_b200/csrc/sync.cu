// Cross-GPU flag signalling with BOUNDED waits, and the CUDA IPC / peer-access plumbing.
//
// A waiting kernel never spins without limit: after `timeout_ns` of device time (and, as a
// second bound, a fixed number of polls) it records AD_ERR_TIMEOUT in a status word and
// returns, so the context stays usable and the host can report the failure.
#include "common.cuh"

namespace adk {

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void flag_wait_kernel(const unsigned long long* flag, unsigned long long epoch, unsigned long long timeout_ns,
                                 int* status) {
  const unsigned long long t0 = global_timer_ns();
  for (unsigned long long polls = 0; polls < (1ull << 28); ++polls) {
    if (ld_acquire_sys(flag) >= epoch) return;
    if (global_timer_ns() - t0 > timeout_ns) break;
    __nanosleep(128);
  }
  if (status) *status = AD_ERR_TIMEOUT;
}

__global__ void flag_signal_kernel(unsigned long long* flag, unsigned long long epoch) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(epoch) : "memory");
}

// The same with the value taken relative to a device-resident base: kernels recorded once (a CUDA graph)
// then work for every step, the base being advanced on the device between steps.
__global__ void flag_wait_rel_kernel(const unsigned long long* flag, const unsigned long long* base, unsigned long long offset,
                                     unsigned long long timeout_ns, int* status) {
  const unsigned long long epoch = *base + offset;
  const unsigned long long t0 = global_timer_ns();
  for (unsigned long long polls = 0; polls < (1ull << 28); ++polls) {
    if (ld_acquire_sys(flag) >= epoch) return;
    if (global_timer_ns() - t0 > timeout_ns) break;
    __nanosleep(128);
  }
  if (status) *status = AD_ERR_TIMEOUT;
}
__global__ void flag_signal_rel_kernel(unsigned long long* flag, const unsigned long long* base, unsigned long long offset) {
  const unsigned long long epoch = *base + offset;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flag), "l"(epoch) : "memory");
}
__global__ void flag_advance_kernel(unsigned long long* base, unsigned long long delta) { *base += delta; }

// out[i] = sum_q bufs[q][i] for i in [begin, end), peers in rank order (float4 body, scalar tail)
struct PeerBufs { const float* p[AD_MAX_PEERS]; };
__global__ void __launch_bounds__(256) peer_sum_kernel(PeerBufs b, uint32_t R, float* out, size_t begin, size_t end) {
  const size_t nt = (size_t)gridDim.x * blockDim.x, tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t a4 = (begin + 3) / 4 * 4, e4 = end / 4 * 4;
  const bool body = a4 < e4;
  const size_t head_end = body ? a4 : end, tail_begin = body ? e4 : end;
  for (size_t i = begin + tid; i < head_end; i += nt) {
    float acc = 0.f;
    for (uint32_t q = 0; q < R; ++q) acc += b.p[q][i];
    out[i] = acc;
  }
  if (body)
    for (size_t i = a4 / 4 + tid; i < e4 / 4; i += nt) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (uint32_t q = 0; q < R; ++q) {
        const float4 v = ((const float4*)b.p[q])[i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      ((float4*)out)[i] = acc;
    }
  for (size_t i = tail_begin + tid; i < end; i += nt) {
    float acc = 0.f;
    for (uint32_t q = 0; q < R; ++q) acc += b.p[q][i];
    out[i] = acc;
  }
}

}  // namespace adk

using namespace adk;

extern "C" int ad_flag_wait_rel(const uint64_t* flag, const uint64_t* base, uint64_t offset, uint64_t timeout_ns,
                                int32_t* status_word, void* stream) {
  if (!flag || !base || !status_word) return AD_ERR_BAD_ARG;
  if (timeout_ns == 0 || timeout_ns > 10000000000ull) return AD_ERR_BAD_ARG;
  flag_wait_rel_kernel<<<1, 1, 0, as_stream(stream)>>>((const unsigned long long*)flag, (const unsigned long long*)base, offset,
                                                       timeout_ns, status_word);
  count_launch();
  return launch_status();
}
extern "C" int ad_flag_signal_rel(uint64_t* flag, const uint64_t* base, uint64_t offset, void* stream) {
  if (!flag || !base) return AD_ERR_BAD_ARG;
  flag_signal_rel_kernel<<<1, 1, 0, as_stream(stream)>>>((unsigned long long*)flag, (const unsigned long long*)base, offset);
  count_launch();
  return launch_status();
}
extern "C" int ad_flag_advance(uint64_t* base, uint64_t delta, void* stream) {
  if (!base) return AD_ERR_BAD_ARG;
  flag_advance_kernel<<<1, 1, 0, as_stream(stream)>>>((unsigned long long*)base, delta);
  count_launch();
  return launch_status();
}
extern "C" int ad_peer_sum(uint32_t num_ranks, const float* const* bufs, float* out, size_t begin, size_t end, void* stream) {
  if (!bufs || !out || num_ranks == 0 || num_ranks > AD_MAX_PEERS || begin > end) return AD_ERR_BAD_ARG;
  if (begin == end) return AD_OK;
  PeerBufs b{};
  for (uint32_t q = 0; q < num_ranks; ++q) {
    if (!bufs[q] || ((uintptr_t)bufs[q] & 15u)) return bufs[q] ? AD_ERR_ALIGN : AD_ERR_BAD_ARG;
    b.p[q] = bufs[q];
  }
  if ((uintptr_t)out & 15u) return AD_ERR_ALIGN;
  peer_sum_kernel<<<grid_for((end - begin + 3) / 4, 256), 256, 0, as_stream(stream)>>>(b, num_ranks, out, begin, end);
  count_launch();
  return launch_status();
}

extern "C" int ad_flag_wait(const uint64_t* flag, uint64_t epoch, uint64_t timeout_ns, int32_t* status_word, void* stream) {
  if (!flag || !status_word) return AD_ERR_BAD_ARG;
  if (timeout_ns == 0 || timeout_ns > 10000000000ull) return AD_ERR_BAD_ARG;  // at most 10 s
  flag_wait_kernel<<<1, 1, 0, as_stream(stream)>>>((const unsigned long long*)flag, epoch, timeout_ns, status_word);
  count_launch();
  return launch_status();
}

extern "C" int ad_flag_signal(uint64_t* flag, uint64_t epoch, void* stream) {
  if (!flag) return AD_ERR_BAD_ARG;
  flag_signal_kernel<<<1, 1, 0, as_stream(stream)>>>((unsigned long long*)flag, epoch);
  count_launch();
  return launch_status();
}

static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");

extern "C" int ad_ipc_get_handle(void* dev_ptr, uint8_t handle_out[64]) {
  if (!dev_ptr || !handle_out) return AD_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, dev_ptr) != cudaSuccess) { cudaGetLastError(); return AD_ERR_CUDA; }
  memcpy(handle_out, &h, 64);
  return AD_OK;
}

extern "C" int ad_ipc_open_handle(const uint8_t handle[64], void** dev_ptr_out) {
  if (!handle || !dev_ptr_out) return AD_ERR_BAD_ARG;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  if (cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return AD_ERR_CUDA;
  }
  return AD_OK;
}

extern "C" int ad_ipc_close_handle(void* dev_ptr) {
  if (!dev_ptr) return AD_ERR_BAD_ARG;
  if (cudaIpcCloseMemHandle(dev_ptr) != cudaSuccess) { cudaGetLastError(); return AD_ERR_CUDA; }
  return AD_OK;
}

extern "C" int ad_enable_peer_access(int device, int peer_device) {
  if (device == peer_device) return AD_OK;
  int can = 0;
  if (cudaDeviceCanAccessPeer(&can, device, peer_device) != cudaSuccess || !can) { cudaGetLastError(); return AD_ERR_UNSUPPORTED; }
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device);
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  cudaSetDevice(prev);
  if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return AD_ERR_CUDA; }
  cudaGetLastError();
  return AD_OK;
}

extern "C" int ad_device_malloc(size_t bytes, void** dev_ptr_out) {
  if (!dev_ptr_out || bytes == 0) return AD_ERR_BAD_ARG;
  if (cudaMalloc(dev_ptr_out, bytes) != cudaSuccess) { cudaGetLastError(); return AD_ERR_CUDA; }
  return AD_OK;
}

extern "C" int ad_device_free(void* dev_ptr) {
  if (!dev_ptr) return AD_ERR_BAD_ARG;
  if (cudaFree(dev_ptr) != cudaSuccess) { cudaGetLastError(); return AD_ERR_CUDA; }
  return AD_OK;
}
