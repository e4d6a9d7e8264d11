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

}  // namespace adk

using namespace adk;

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
