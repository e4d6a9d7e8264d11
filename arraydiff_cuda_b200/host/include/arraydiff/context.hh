// Device and communicator set-up of the op-graph API: Context, GPUConn, GPUContext,
// MultiGPUContext.  Same classes and methods as the reference's include/arraydiff/context.hh:23-104
// (bodies src/context.cc:21-158), with three differences that the B200 design needs:
//   * no cuBLAS / cuDNN handles -- every op calls the arraydiff_b200 C ABI;
//   * each rank owns ONE device arena; GPUMemory sub-allocates from it in graph-build order, so a
//     buffer sits at the same offset on every rank and peers are reached as peer_base + offset
//     (same process: direct pointers; one process per GPU: bases opened from CUDA IPC handles);
//   * ranks may share a device ("virtual ranks"), so a 1 x R strip grid can be exercised on one GPU,
//     and a device subset can be chosen (the reference always takes every visible device,
//     src/context.cc:117-134).
#ifndef ARRAYDIFF_CONTEXT_HH
#define ARRAYDIFF_CONTEXT_HH

#include <cuda_runtime.h>

#include <cassert>
#include <functional>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <vector>

#include "arraydiff_b200.h"

namespace arraydiff {

using std::shared_ptr;
using std::vector;

template <typename T> class GPUMemory;
class Spatial2DComm;

// How activations are stored and which kernels run: fp32 NCHW (the reference's layout, exact
// fp32 FMA kernels) or bf16 NHWC (tensor-core kernels, fp32 accumulate).
enum ComputeMode { COMPUTE_F32_NCHW = 0, COMPUTE_BF16_NHWC = 1 };

class Context {
public:
  virtual ~Context() {}
  virtual void sync() = 0;
};

// Scoped "current device": sets the device on construction, restores the previous one on
// destruction (reference: src/context.cc:23-38).
class GPUConn {
public:
  GPUConn(int device, cudaStream_t stream);
  ~GPUConn();
  GPUConn(const GPUConn&) = delete;
  GPUConn(GPUConn&& o) : device_(o.device_), prev_(o.prev_), stream_(o.stream_), owner_(o.owner_) { o.owner_ = false; }
  int device() const { return device_; }
  cudaStream_t stream() { return stream_; }
  void sync();
private:
  int device_, prev_;
  cudaStream_t stream_;
  bool owner_;
};

// Bump allocator over one cudaMalloc'd block; never frees (as GPUMemory in the reference,
// include/arraydiff/array_gpu.hh:82-109).
class DeviceArena {
public:
  DeviceArena() : base_(nullptr), bytes_(0), used_(0) {}
  void init(size_t bytes);
  void* alloc(size_t bytes, size_t align = 1024);
  uint8_t* base() const { return base_; }
  size_t used() const { return used_; }
  size_t capacity() const { return bytes_; }
private:
  uint8_t* base_;
  size_t bytes_, used_;
};

class GPUContext : public virtual Context {
public:
  static shared_ptr<GPUContext> Make(int device);
  explicit GPUContext(int device, size_t arena_bytes = 0);
  virtual ~GPUContext();
  virtual void sync();
  // Scoped access to this rank's device and stream.  Work that was deferred on the stream (set_pending: the waits for the
  // neighbours' halo rows of the last exchange) is issued first, so that whatever the caller launches next sees the
  // halo rows; conn_deferred() skips that step for a caller that launches work which does not read them and then calls
  // finish_pending() itself (the convolution operator: interior rows, wait, boundary rows).
  GPUConn conn();
  GPUConn conn_deferred();
  void set_pending(std::function<void(cudaStream_t)> f) { finish_pending(); pending_ = f; }
  bool has_pending() const { return (bool)pending_; }
  void finish_pending();
  int device() const { return device_; }
  cudaStream_t stream() const { return stream_; }
  DeviceArena& arena() { return arena_; }
  ComputeMode mode() const { return mode_; }
  void set_mode(ComputeMode m) { mode_ = m; }
  // Growable scratch workspace (reference: src/context.cc:76-100).
  void reserve_scratch(size_t min_scratch_size);
  void* get_scratch() { return scratch_; }
  size_t scratch_size() const { return scratch_size_; }
  int32_t* status_word() { return status_; }   // device word that bounded waits report into
  int read_status();                            // synchronises this rank's stream
  // Side stream for work whose result nothing needs before the end of the backward walk (the filter gradients: they run
  // underneath the memory-bound operators of the layers below).  fork_side() orders the side stream after everything
  // issued on the main stream so far and returns it; join_side() orders the main stream after the side stream's work.
  // Op::backward() ends with JoinAllSides(), so every consumer of a gradient sees it complete; inside a stream capture
  // the side stream joins the capture at the fork and leaves it at the join.
  cudaStream_t fork_side();
  void join_side();
  static void JoinAllSides();
  void reserve_side_scratch(size_t min_size);
  void* side_scratch() { return side_scratch_; }
  size_t side_scratch_size() const { return side_scratch_size_; }
private:
  cudaStream_t side_ = nullptr;
  cudaEvent_t fork_ev_ = nullptr, join_ev_ = nullptr;
  bool side_dirty_ = false;
  void* side_scratch_ = nullptr;
  size_t side_scratch_size_ = 0;
  int device_;
  cudaStream_t stream_;
  DeviceArena arena_;
  ComputeMode mode_;
  void* scratch_;
  size_t scratch_size_;
  int32_t* status_;
  std::function<void(cudaStream_t)> pending_;
};

class MultiGPUContext : public virtual Context {
public:
  // One rank per visible device (the reference's behaviour), or per entry of
  // ARRAYDIFF_B200_DEVICES="0,0,1,1" when that variable is set.
  static shared_ptr<MultiGPUContext> Make();
  // One rank per entry of `devices`; entries may repeat (several strips on one GPU).
  static shared_ptr<MultiGPUContext> Make(const vector<int>& devices, ComputeMode mode = COMPUTE_F32_NCHW,
                                          size_t arena_bytes_per_rank = 0);
  // One process per GPU: this process is `rank` of `num_ranks`; peers' arena bases are supplied
  // afterwards with set_peer_arena() (pointers from ad_ipc_open_handle).
  static shared_ptr<MultiGPUContext> MakeDistributed(size_t rank, size_t num_ranks, int device, ComputeMode mode,
                                                     size_t arena_bytes);
  MultiGPUContext(const vector<int>& devices, ComputeMode mode, size_t arena_bytes, bool distributed, size_t my_rank,
                  size_t num_ranks);
  virtual ~MultiGPUContext() {}

  virtual void sync();
  void sync_rank(size_t rank);
  size_t num_ranks() const { return num_ranks_; }
  bool distributed() const { return distributed_; }
  bool is_local(size_t rank) const { return distributed_ ? rank == my_rank_ : true; }
  size_t my_rank() const { return my_rank_; }
  ComputeMode mode() const { return mode_; }

  shared_ptr<GPUContext> device_context(size_t rank);
  Spatial2DComm* spatial_comm(size_t rank);
  // Base address of rank r's arena as seen from this process.
  uint8_t* arena_base(size_t rank) const { return arena_bases_.at(rank); }
  void set_peer_arena(size_t rank, void* base) { arena_bases_.at(rank) = (uint8_t*)base; }
  // The same allocation on rank r: translate a pointer inside `from_rank`'s arena.
  void* peer_ptr(const void* p, size_t from_rank, size_t to_rank) const {
    return arena_bases_.at(to_rank) + ((const uint8_t*)p - arena_bases_.at(from_rank));
  }
  // Sum of one fp32 buffer (same arena offset on every rank) over all ranks, result on every rank:
  // the weight-gradient allreduce.  In-process ranks add through peer pointers; between processes
  // the caller-installed hook (NCCL) is used.
  typedef void (*AllreduceHook)(float* buf, size_t count, cudaStream_t stream, void* user);
  void set_allreduce_hook(AllreduceHook fn, void* user) { ar_hook_ = fn; ar_user_ = user; }
  bool has_allreduce_hook() const { return ar_hook_ != nullptr; }
  void allreduce_sum(float* local_buf_rank0_offset_base, size_t count);
  // Data-parallel replicas around the spatial group (one process per GPU): this process is `world_rank` of
  // `world_size` processes that all hold the same net, so the same allocation sits at the same arena offset in
  // each; their arena bases are supplied with set_world_peer_arena().  The built-in gradient exchange then sums
  // over all of them instead of over the spatial group only (4 data groups x 2 strips = 8 processes).
  void set_world(size_t world_rank, size_t world_size) {
    world_rank_ = world_rank; world_size_ = world_size;
    world_bases_.assign(world_size, nullptr);
    world_bases_.at(world_rank) = arena_bases_.at(my_rank_);
  }
  void set_world_peer_arena(size_t world_rank, void* base) { world_bases_.at(world_rank) = (uint8_t*)base; }
  // this process's place in the gradient exchange: the world when set_world() was called, else the spatial group
  size_t exchange_rank() const { return world_size_ ? world_rank_ : my_rank_; }
  size_t exchange_size() const { return world_size_ ? world_size_ : num_ranks_; }
  // Communicator handles for callers that run NCCL themselves (the reference's nccl_comm(rank),
  // include/arraydiff/context.hh:92): opaque here -- this library never calls NCCL; whoever initialises the
  // communicators hands them over with set_nccl_comm and reads them back (cast to ncclComm_t) inside an allreduce hook.
  void set_nccl_comm(size_t rank, void* comm) { if (nccl_comms_.size() < num_ranks_) nccl_comms_.resize(num_ranks_, nullptr); nccl_comms_.at(rank) = comm; }
  void* nccl_comm(size_t rank) const { return rank < nccl_comms_.size() ? nccl_comms_[rank] : nullptr; }
  // Between processes: advances every local rank's flag base by the signalling operations issued since the
  // last call (Spatial2DComm::end_phase).  Call it where a unit of work that may be replayed as a CUDA graph ends.
  void end_phase();

private:
  size_t num_ranks_, my_rank_;
  bool distributed_;
  ComputeMode mode_;
  vector<shared_ptr<GPUContext>> dev_ctxs_;   // indexed by rank; null for remote ranks
  vector<uint8_t*> arena_bases_;
  Spatial2DComm* spatial_comms_;
  AllreduceHook ar_hook_;
  void* ar_user_;
  float* ar_stage_ = nullptr;    // between processes without a hook: this rank's gradient as its peers read it
  size_t ar_stage_count_ = 0;
  size_t world_rank_ = 0, world_size_ = 0;   // 0: the gradient exchange spans the spatial group
  vector<uint8_t*> world_bases_;
  vector<void*> nccl_comms_;
};

}  // namespace arraydiff
#endif
