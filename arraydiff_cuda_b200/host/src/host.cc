// Context, arena, Spatial2DComm, arrays and the op-graph walk of the host layer.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "arraydiff/op.hh"

namespace arraydiff {

[[noreturn]] void ad_fail(int status, const char* what, const char* file, int line) {
  std::fprintf(stderr, "arraydiff: %s failed: %s (%d) at %s:%d\n", what, ad_status_string(status), status, file, line);
  std::abort();
}
[[noreturn]] void cuda_fail(int err, const char* what, const char* file, int line) {
  std::fprintf(stderr, "arraydiff: %s failed: %s at %s:%d\n", what, cudaGetErrorString((cudaError_t)err), file, line);
  std::abort();
}

// ------------------------------------------------------------------ GPUConn / arena / contexts
GPUConn::GPUConn(int device, cudaStream_t stream) : device_(device), prev_(0), stream_(stream), owner_(true) {
  CUDA_CHECK(cudaGetDevice(&prev_));
  if (prev_ != device_) CUDA_CHECK(cudaSetDevice(device_));
}
GPUConn::~GPUConn() {
  if (owner_ && prev_ != device_) cudaSetDevice(prev_);
}
void GPUConn::sync() { CUDA_CHECK(cudaStreamSynchronize(stream_)); }

void DeviceArena::init(size_t bytes) {
  void* p = nullptr;
  AD_CHECK(ad_device_malloc(bytes, &p));
  base_ = (uint8_t*)p;
  bytes_ = bytes;
  used_ = 0;
}
void* DeviceArena::alloc(size_t bytes, size_t align) {
  size_t off = (used_ + align - 1) / align * align;
  if (off + bytes > bytes_) {
    std::fprintf(stderr, "arraydiff: device arena exhausted (%zu + %zu > %zu); raise ARRAYDIFF_B200_ARENA_MB\n", off, bytes, bytes_);
    std::abort();
  }
  used_ = off + bytes;
  return base_ + off;
}

static size_t default_arena_bytes() {
  const char* e = std::getenv("ARRAYDIFF_B200_ARENA_MB");
  size_t mb = e ? (size_t)std::atoll(e) : 2048;
  return mb << 20;
}

// contexts of this process, for JoinAllSides (the host layer is driven by one thread per process)
static std::vector<GPUContext*>& all_contexts() { static std::vector<GPUContext*> v; return v; }
shared_ptr<GPUContext> GPUContext::Make(int device) { return make_shared<GPUContext>(device); }

GPUContext::GPUContext(int device, size_t arena_bytes)
    : device_(device), stream_(nullptr), mode_(COMPUTE_F32_NCHW), scratch_(nullptr), scratch_size_(0), status_(nullptr) {
  int prev = 0;
  CUDA_CHECK(cudaGetDevice(&prev));
  CUDA_CHECK(cudaSetDevice(device_));
  // the main stream outranks the side stream (fork_side): where both have blocks ready, the critical path goes first
  int least = 0, greatest = 0;
  CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
  CUDA_CHECK(cudaStreamCreateWithPriority(&stream_, cudaStreamNonBlocking, greatest));
  arena_.init(arena_bytes ? arena_bytes : default_arena_bytes());
  status_ = (int32_t*)arena_.alloc(64);
  CUDA_CHECK(cudaMemsetAsync(status_, 0, 64, stream_));
  CUDA_CHECK(cudaSetDevice(prev));
  all_contexts().push_back(this);
}
GPUContext::~GPUContext() {
  auto& v = all_contexts();
  v.erase(std::remove(v.begin(), v.end(), this), v.end());
}
cudaStream_t GPUContext::fork_side() {
  GPUConn c(device_, stream_);
  if (!side_) {
    int least = 0, greatest = 0;
    CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    CUDA_CHECK(cudaStreamCreateWithPriority(&side_, cudaStreamNonBlocking, least));
    CUDA_CHECK(cudaEventCreateWithFlags(&fork_ev_, cudaEventDisableTiming));
    CUDA_CHECK(cudaEventCreateWithFlags(&join_ev_, cudaEventDisableTiming));
  }
  CUDA_CHECK(cudaEventRecord(fork_ev_, stream_));
  CUDA_CHECK(cudaStreamWaitEvent(side_, fork_ev_, 0));
  side_dirty_ = true;
  return side_;
}
void GPUContext::join_side() {
  if (!side_dirty_) return;
  GPUConn c(device_, stream_);
  CUDA_CHECK(cudaEventRecord(join_ev_, side_));
  CUDA_CHECK(cudaStreamWaitEvent(stream_, join_ev_, 0));
  side_dirty_ = false;
}
void GPUContext::JoinAllSides() {
  for (GPUContext* g : all_contexts()) g->join_side();
}
void GPUContext::reserve_side_scratch(size_t min_size) {
  if (side_scratch_size_ >= min_size) return;
  size_t want = min_size < (1u << 20) ? (1u << 20) : min_size;
  side_scratch_ = arena_.alloc(want);
  side_scratch_size_ = want;
}
void GPUContext::sync() { join_side(); GPUConn c = conn(); c.sync(); }
GPUConn GPUContext::conn() {
  GPUConn c(device_, stream_);
  finish_pending();
  return c;
}
GPUConn GPUContext::conn_deferred() { return GPUConn(device_, stream_); }
void GPUContext::finish_pending() {
  if (!pending_) return;
  auto f = pending_;
  pending_ = nullptr;
  f(stream_);   // issued with this context's device current: callers hold a GPUConn
}
void GPUContext::reserve_scratch(size_t min_scratch_size) {
  if (scratch_size_ >= min_scratch_size) return;
  size_t want = min_scratch_size < (1u << 20) ? (1u << 20) : min_scratch_size;
  scratch_ = arena_.alloc(want);
  scratch_size_ = want;
}
int GPUContext::read_status() {
  GPUConn c = conn();
  int32_t v = 0;
  CUDA_CHECK(cudaMemcpyAsync(&v, status_, 4, cudaMemcpyDeviceToHost, c.stream()));
  c.sync();
  return v;
}

shared_ptr<MultiGPUContext> MultiGPUContext::Make() {
  vector<int> devs;
  if (const char* e = std::getenv("ARRAYDIFF_B200_DEVICES")) {
    std::stringstream ss(e);
    string tok;
    while (std::getline(ss, tok, ',')) devs.push_back(std::atoi(tok.c_str()));
  } else {
    int n = 0;
    CUDA_CHECK(cudaGetDeviceCount(&n));
    for (int i = 0; i < n; ++i) devs.push_back(i);
  }
  // ARRAYDIFF_B200_MODE=bf16 selects the tensor-core path (default: the reference's fp32 NCHW arithmetic);
  // ARRAYDIFF_B200_ARENA_MB sizes each rank's arena
  ComputeMode mode = COMPUTE_F32_NCHW;
  if (const char* m = std::getenv("ARRAYDIFF_B200_MODE")) if (!std::strcmp(m, "bf16")) mode = COMPUTE_BF16_NHWC;
  size_t arena = 0;
  if (const char* a = std::getenv("ARRAYDIFF_B200_ARENA_MB")) arena = (size_t)std::strtoull(a, nullptr, 10) << 20;
  return Make(devs, mode, arena);
}
shared_ptr<MultiGPUContext> MultiGPUContext::Make(const vector<int>& devices, ComputeMode mode, size_t arena_bytes) {
  return make_shared<MultiGPUContext>(devices, mode, arena_bytes, false, 0, devices.size());
}
shared_ptr<MultiGPUContext> MultiGPUContext::MakeDistributed(size_t rank, size_t num_ranks, int device, ComputeMode mode,
                                                             size_t arena_bytes) {
  return make_shared<MultiGPUContext>(vector<int>{device}, mode, arena_bytes, true, rank, num_ranks);
}

MultiGPUContext::MultiGPUContext(const vector<int>& devices, ComputeMode mode, size_t arena_bytes, bool distributed,
                                 size_t my_rank, size_t num_ranks)
    : num_ranks_(num_ranks), my_rank_(my_rank), distributed_(distributed), mode_(mode), ar_hook_(nullptr), ar_user_(nullptr) {
  assert(num_ranks_ >= 1 && num_ranks_ <= ARRAYDIFF_MAX_PEERS);
  dev_ctxs_.resize(num_ranks_);
  arena_bases_.assign(num_ranks_, nullptr);
  for (size_t r = 0; r < num_ranks_; ++r) {
    if (!is_local(r)) continue;
    int dev = distributed_ ? devices.at(0) : devices.at(r);
    dev_ctxs_[r] = make_shared<GPUContext>(dev, arena_bytes);
    dev_ctxs_[r]->set_mode(mode);
    arena_bases_[r] = dev_ctxs_[r]->arena().base();
  }
  if (!distributed_)
    for (size_t a = 0; a < num_ranks_; ++a)
      for (size_t b = 0; b < num_ranks_; ++b)
        if (devices[a] != devices[b]) AD_CHECK(ad_enable_peer_access(devices[a], devices[b]));   // reference src/spatial.cc:13-29
  spatial_comms_ = new Spatial2DComm[num_ranks_];
  Spatial2DComm::InitAll(spatial_comms_, 1, (uint32_t)num_ranks_, this);                        // reference src/context.cc:134
}
void MultiGPUContext::sync() {
  for (size_t r = 0; r < num_ranks_; ++r) if (dev_ctxs_[r]) dev_ctxs_[r]->sync();
}
void MultiGPUContext::end_phase() {
  if (!distributed_) return;
  for (size_t r = 0; r < num_ranks_; ++r)
    if (is_local(r)) {
      GPUConn c = dev_ctxs_[r]->conn();     // issues waits still pending on the rank: they use this phase's values
      spatial_comms_[r].end_phase(c.stream());
    }
}
void MultiGPUContext::sync_rank(size_t rank) { dev_ctxs_.at(rank)->sync(); }
shared_ptr<GPUContext> MultiGPUContext::device_context(size_t rank) { assert(dev_ctxs_.at(rank)); return dev_ctxs_.at(rank); }
Spatial2DComm* MultiGPUContext::spatial_comm(size_t rank) { return &spatial_comms_[rank]; }

void MultiGPUContext::allreduce_sum(float* buf, size_t count) {
  if (num_ranks_ == 1 && world_size_ <= 1 && !(distributed_ && ar_hook_)) return;
  if (distributed_ && ar_hook_) {
    ar_hook_(buf, count, dev_ctxs_[my_rank_]->stream(), ar_user_);   // e.g. ncclAllReduce
    return;
  }
  if (distributed_) {
    // No hook: reduce-scatter + all-gather with peer loads, ordered by flag words with bounded waits.  Every
    // kernel and copy is on this rank's stream and every flag value is relative, so the whole exchange can be
    // captured in a CUDA graph; each slice is summed once, in rank order, so all ranks end with the same bits.
    // the exchange spans the spatial group, or all data-parallel replicas when set_world() was called
    const bool wide = world_size_ > 0;
    const size_t r = wide ? world_rank_ : my_rank_, R = wide ? world_size_ : num_ranks_;
    GPUContext* g = dev_ctxs_[my_rank_].get();
    GPUConn conn = g->conn();
    cudaStream_t s = conn.stream();
    Spatial2DComm* comm = &spatial_comms_[my_rank_];
    uint8_t* my_base = arena_bases_.at(my_rank_);
    auto at = [&](const void* p, size_t q) -> void* {      // the same allocation in participant q's arena
      uint8_t* base = wide ? world_bases_.at(q) : arena_bases_.at(q);
      assert(base && "peer arena not set");
      return base + ((const uint8_t*)p - my_base);
    };
    if (ar_stage_count_ < count) {
      ar_stage_ = (float*)g->arena().alloc(count * sizeof(float));   // same offset on every rank: all ranks get here alike
      ar_stage_count_ = count;
    }
    const uint64_t kTimeoutNs = 2000000000ull;
    auto round = [&]() {
      const uint64_t k = comm->next_phase_epoch();
      for (size_t q = 0; q < R; ++q)
        if (q != r) AD_CHECK(ad_flag_signal_rel((uint64_t*)at(comm->allreduce_flags() + r, q), comm->epoch_base(), k, s));
      for (size_t q = 0; q < R; ++q)
        if (q != r) AD_CHECK(ad_flag_wait_rel(comm->allreduce_flags() + q, comm->epoch_base(), k, kTimeoutNs, g->status_word(), s));
    };
    CUDA_CHECK(cudaMemcpyAsync(ar_stage_, buf, count * sizeof(float), cudaMemcpyDeviceToDevice, s));
    round();                                                       // every rank's staged gradient is readable
    const size_t per = ((count + R - 1) / R + 3) / 4 * 4;
    auto lo = [&](size_t q) { return std::min(count, q * per); };
    const float* srcs[ARRAYDIFF_MAX_PEERS];
    for (size_t q = 0; q < R; ++q) srcs[q] = (const float*)at(ar_stage_, q);
    AD_CHECK(ad_peer_sum((uint32_t)R, srcs, buf, lo(r), lo(r + 1), s));   // my slice of the sum
    round();                                                       // every rank's slice is final
    for (size_t q = 0; q < R; ++q) {
      if (q == r || lo(q) == lo(q + 1)) continue;
      CUDA_CHECK(cudaMemcpyAsync(buf + lo(q), (const float*)at(buf, q) + lo(q), (lo(q + 1) - lo(q)) * sizeof(float),
                                 cudaMemcpyDeviceToDevice, s));
    }
    round();                                                       // nobody still reads my slice or my staged copy
    return;
  }
  // In-process ranks: rank 0 adds every peer's buffer (peer loads), then every peer copies the sum back.
  vector<cudaEvent_t> ev(num_ranks_);
  for (size_t r = 0; r < num_ranks_; ++r) {
    GPUConn c = dev_ctxs_[r]->conn();
    CUDA_CHECK(cudaEventCreateWithFlags(&ev[r], cudaEventDisableTiming));
    CUDA_CHECK(cudaEventRecord(ev[r], c.stream()));
  }
  cudaEvent_t done;
  {
    GPUConn c = dev_ctxs_[0]->conn();
    for (size_t r = 1; r < num_ranks_; ++r) {
      CUDA_CHECK(cudaStreamWaitEvent(c.stream(), ev[r], 0));
      AD_CHECK(ad_array_add(count, (const float*)peer_ptr(buf, 0, r), buf, c.stream()));
    }
    CUDA_CHECK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    CUDA_CHECK(cudaEventRecord(done, c.stream()));
  }
  for (size_t r = 1; r < num_ranks_; ++r) {
    GPUConn c = dev_ctxs_[r]->conn();
    CUDA_CHECK(cudaStreamWaitEvent(c.stream(), done, 0));
    CUDA_CHECK(cudaMemcpyAsync(peer_ptr(buf, 0, r), buf, count * sizeof(float), cudaMemcpyDeviceToDevice, c.stream()));
    // rank 0 goes on to update its buffer in place (the SGD kernel adds the L2 term into the gradient):
    // not before every peer has taken its copy
    CUDA_CHECK(cudaEventRecord(ev[r], c.stream()));
  }
  {
    GPUConn c = dev_ctxs_[0]->conn();
    for (size_t r = 1; r < num_ranks_; ++r) CUDA_CHECK(cudaStreamWaitEvent(c.stream(), ev[r], 0));
  }
  for (auto e : ev) cudaEventDestroy(e);
  cudaEventDestroy(done);
}

// ------------------------------------------------------------------ Spatial2DComm
void Spatial2DComm::InitAll(Spatial2DComm* comms, uint32_t num_w_ranks, uint32_t num_h_ranks) {
  InitAll(comms, num_w_ranks, num_h_ranks, nullptr);
}
void Spatial2DComm::InitAll(Spatial2DComm* comms, uint32_t num_w_ranks, uint32_t num_h_ranks, MultiGPUContext* ctx) {
  // rank = rank_h * num_w_ranks + rank_w (row-major over the grid).  1 x R grids (H-strips) work inside one process and
  // between processes; grids with num_w_ranks > 1 (W-split, 2 x 2, 2 x 4 ...; reference src/spatial.cc:105-131,
  // :166-196 for 2 x 1) inside one process.
  assert((num_w_ranks == 1 || !ctx || !ctx->distributed()) && "grids with a W split are built for one-process contexts");
  const uint32_t R = num_w_ranks * num_h_ranks;
  assert(R >= 1 && R <= ARRAYDIFF_MAX_PEERS);
  for (uint32_t r = 0; r < R; ++r) {
    Spatial2DComm& c = comms[r];
    c.rank = r; c.rank_w = r % num_w_ranks; c.rank_h = r / num_w_ranks;
    c.num_ranks = R; c.num_w_ranks = num_w_ranks; c.num_h_ranks = num_h_ranks;
    c.epoch = 0;
    c.ctx_ = ctx;
    for (uint32_t q = 0; q < ARRAYDIFF_MAX_PEERS; ++q) c.peer_comms[q] = q < R ? &comms[q] : nullptr;
    if (ctx && ctx->is_local(r)) {
      auto g = ctx->device_context(r);
      GPUConn conn = g->conn();
      CUDA_CHECK(cudaEventCreateWithFlags(&c.ready_, cudaEventDisableTiming));
      c.flags_ = (uint64_t*)g->arena().alloc(64);      // same offset on every rank: first allocation after the status word
      c.counter_ = (uint32_t*)g->arena().alloc(64);
      c.gflags_ = (uint64_t*)g->arena().alloc(64);
      c.arflags_ = (uint64_t*)g->arena().alloc(64);
      c.ebase_ = (uint64_t*)g->arena().alloc(64);
      CUDA_CHECK(cudaMemsetAsync(c.gflags_, 0, 64, conn.stream()));
      CUDA_CHECK(cudaMemsetAsync(c.arflags_, 0, 64, conn.stream()));
      CUDA_CHECK(cudaMemsetAsync(c.ebase_, 0, 64, conn.stream()));
      CUDA_CHECK(cudaMemsetAsync(c.flags_, 0, 64, conn.stream()));
      CUDA_CHECK(cudaMemsetAsync(c.counter_, 0, 64, conn.stream()));
      conn.sync();
    }
  }
}

void Spatial2DComm::group_start() { in_group_ = true; }
void Spatial2DComm::end_phase(cudaStream_t s) {
  if (!ebase_ || phase_ == 0) return;
  AD_CHECK(ad_flag_advance(ebase_, phase_, s));
  phase_ = 0;
}

void Spatial2DComm::record(Spatial2DOperation op, void* buf, uint32_t p, uint32_t w, uint32_t h, uint32_t c, uint32_t n,
                           Spatial2DTensorFormat f, Spatial2DDataType t) {
  assert(in_group_ && "halo_* must be called between group_start and group_end");
  arg.operation = op; arg.tensor_format = f; arg.data_type = t;
  arg.halo_pad = p; arg.base_width = w; arg.base_height = h; arg.num_channels = c; arg.batch_size = n;
  arg.buffer = buf;
  ++epoch;
  arg.epoch = epoch;
  if (!ctx_) return;
  auto g = ctx_->device_context(rank);
  GPUConn conn = g->conn();
  if (!ctx_->distributed()) {
    // "my buffer is as my neighbours may now read it"
    CUDA_CHECK(cudaEventRecord(ready_, conn.stream()));
    return;
  }
  const uint64_t k = next_phase_epoch();   // between processes: the value is *epoch_base() + k
  arg.epoch = k;
  if (op == SPATIAL2D_OP_HXEXCH) {
    // my padded buffer exists, its pad cells are zeroed and its interior is written: the neighbours
    // may now push into my halo rows (words 4 / 5: "next is ready" / "prev is ready")
    if (rank > 0) AD_CHECK(ad_flag_signal_rel((uint64_t*)ctx_->peer_ptr(flags_ + 4, rank, rank - 1), ebase_, k, conn.stream()));
    if (rank + 1 < num_ranks) AD_CHECK(ad_flag_signal_rel((uint64_t*)ctx_->peer_ptr(flags_ + 5, rank, rank + 1), ebase_, k, conn.stream()));
  } else if (op == SPATIAL2D_OP_HXREDUCE) {
    // my halo-gradient rows are final: tell the neighbours that will pull them
    if (rank + 1 < num_ranks) AD_CHECK(ad_flag_signal_rel((uint64_t*)ctx_->peer_ptr(flags_ + 2, rank, rank + 1), ebase_, k, conn.stream()));
    if (rank > 0) AD_CHECK(ad_flag_signal_rel((uint64_t*)ctx_->peer_ptr(flags_ + 3, rank, rank - 1), ebase_, k, conn.stream()));
  }
}
void Spatial2DComm::halo_exchange(void* buf, uint32_t halo_pad, uint32_t base_width, uint32_t base_height,
                                  uint32_t num_channels, uint32_t batch_size, Spatial2DTensorFormat tensor_format,
                                  Spatial2DDataType data_type) {
  record(SPATIAL2D_OP_HXEXCH, buf, halo_pad, base_width, base_height, num_channels, batch_size, tensor_format, data_type);
}
void Spatial2DComm::halo_reduce(void* buf, uint32_t halo_pad, uint32_t base_width, uint32_t base_height,
                                uint32_t num_channels, uint32_t batch_size, Spatial2DTensorFormat tensor_format,
                                Spatial2DDataType data_type) {
  record(SPATIAL2D_OP_HXREDUCE, buf, halo_pad, base_width, base_height, num_channels, batch_size, tensor_format, data_type);
}

void Spatial2DComm::group_end(GPUConn& conn) {
  assert(in_group_);
  in_group_ = false;
  if (num_ranks == 1 || arg.halo_pad == 0) return;
  ad_halo_args a = {};
  a.dtype = arg.data_type == SPATIAL2D_DATA_FLOAT ? AD_F32 : AD_BF16;
  assert(arg.data_type == SPATIAL2D_DATA_FLOAT || arg.data_type == SPATIAL2D_DATA_BFLOAT16);
  a.layout = arg.tensor_format == SPATIAL2D_TENSOR_NCHW ? AD_NCHW : AD_NHWC;
  a.halo_pad = arg.halo_pad; a.base_width = arg.base_width; a.base_height = arg.base_height;
  a.num_channels = arg.num_channels; a.batch_size = arg.batch_size;
  a.num_ranks = num_ranks; a.rank_first = rank; a.rank_count = 1;
  const bool dist = ctx_ && ctx_->distributed();
  for (uint32_t q = 0; q < num_ranks; ++q) {
    if (dist) {
      a.bufs[q] = ctx_->peer_ptr(arg.buffer, rank, q);
    } else {
      // every rank of the group has recorded its block in this epoch (the reference spins for this, src/spatial.cc:59-70)
      assert(peer_comms[q]->arg.epoch == arg.epoch && peer_comms[q]->arg.operation == arg.operation);
      a.bufs[q] = peer_comms[q]->arg.buffer;
    }
  }
  cudaStream_t s = conn.stream();
  if (num_w_ranks > 1) {
    // 2-D grid (one process): pull from the up-to-8 neighbours once each has handed its buffer over
    assert(!dist);
    ad_halo2d_args b = {};
    b.dtype = a.dtype; b.layout = a.layout;
    b.halo_pad = arg.halo_pad; b.base_width = arg.base_width; b.base_height = arg.base_height;
    b.num_channels = arg.num_channels; b.batch_size = arg.batch_size;
    b.grid_w = num_w_ranks; b.grid_h = num_h_ranks; b.rank_first = rank; b.rank_count = 1; b.push = 0;
    for (uint32_t q = 0; q < num_ranks; ++q) b.bufs[q] = a.bufs[q];
    for (int dy = -1; dy <= 1; ++dy)
      for (int dx = -1; dx <= 1; ++dx) {
        const int ny = (int)rank_h + dy, nx = (int)rank_w + dx;
        if ((!dy && !dx) || ny < 0 || nx < 0 || ny >= (int)num_h_ranks || nx >= (int)num_w_ranks) continue;
        Spatial2DComm* q = peer_comms[(uint32_t)ny * num_w_ranks + (uint32_t)nx];
        if (q->ready_) CUDA_CHECK(cudaStreamWaitEvent(s, q->ready_, 0));
      }
    if (arg.operation == SPATIAL2D_OP_HXEXCH) AD_CHECK(ad_halo2d_exchange(&b, s));
    else AD_CHECK(ad_halo2d_reduce(&b, s));
    return;
  }
  if (!dist) {
    // Pull: my kernel reads my neighbours' rows once they have handed their buffers over.
    if (rank > 0 && peer_comms[rank - 1]->ready_) CUDA_CHECK(cudaStreamWaitEvent(s, peer_comms[rank - 1]->ready_, 0));
    if (rank + 1 < num_ranks && peer_comms[rank + 1]->ready_) CUDA_CHECK(cudaStreamWaitEvent(s, peer_comms[rank + 1]->ready_, 0));
    a.push = 0;
    if (arg.operation == SPATIAL2D_OP_HXEXCH) AD_CHECK(ad_halo_exchange(&a, s));
    else AD_CHECK(ad_halo_reduce(&a, s));
    return;
  }
  auto g = ctx_->device_context(rank);
  const uint64_t kTimeoutNs = 2000000000ull;
  if (arg.operation == SPATIAL2D_OP_HXEXCH) {
    // Push my edge rows into the neighbours' halo rows and publish; then wait for theirs.
    a.push = 1;
    if (rank + 1 < num_ranks) a.signal_flags[rank + 1] = (uint64_t*)ctx_->peer_ptr(flags_ + 0, rank, rank + 1);
    if (rank > 0) a.signal_flags[rank - 1] = (uint64_t*)ctx_->peer_ptr(flags_ + 1, rank, rank - 1);
    a.epoch = arg.epoch;
    a.epoch_base = ebase_;
    a.block_counter = counter_;
    if (rank + 1 < num_ranks) AD_CHECK(ad_flag_wait_rel(flags_ + 4, ebase_, arg.epoch, kTimeoutNs, g->status_word(), s));
    if (rank > 0) AD_CHECK(ad_flag_wait_rel(flags_ + 5, ebase_, arg.epoch, kTimeoutNs, g->status_word(), s));
    AD_CHECK(ad_halo_exchange(&a, s));
    // The waits for the neighbours' rows are left pending on the rank's context: they are issued in front of the next
    // launch that goes through GPUContext::conn() -- or, by a consumer that knows which of its work needs the halo
    // rows (the convolution: interior rows first), after that work.
    const uint64_t ep = arg.epoch;
    uint64_t* const fl = flags_;
    uint64_t* const eb = ebase_;
    int32_t* const st = g->status_word();
    const bool has_prev = rank > 0, has_next = rank + 1 < num_ranks;
    g->set_pending([=](cudaStream_t ws) {
      if (has_prev) AD_CHECK(ad_flag_wait_rel(fl + 0, eb, ep, kTimeoutNs, st, ws));
      if (has_next) AD_CHECK(ad_flag_wait_rel(fl + 1, eb, ep, kTimeoutNs, st, ws));
    });
  } else {
    if (rank > 0) AD_CHECK(ad_flag_wait_rel(flags_ + 2, ebase_, arg.epoch, kTimeoutNs, g->status_word(), s));
    if (rank + 1 < num_ranks) AD_CHECK(ad_flag_wait_rel(flags_ + 3, ebase_, arg.epoch, kTimeoutNs, g->status_word(), s));
    AD_CHECK(ad_halo_reduce(&a, s));
  }
}

// ------------------------------------------------------------------ arrays
template <>
void GPUMemory<float>::set_constant(float c, GPUConn& conn) { AD_CHECK(ad_array_set_constant(size_, c, dptr_, conn.stream())); }

template <>
GPUBatchArray3D<float> GPUBatchArray3D<float>::ZerosPadded(Shape3D dim, Shape3D offset, Shape3D stride, size_t batch,
                                                           GPUContext* ctx) {
  GPUBatchArray3D<float> a;
  a.dim_ = dim; a.offset_ = offset; a.stride_ = stride;
  a.batch_cap_ = a.batch_ = batch;
  a.storage_ = ctx->mode();
  assert(offset.shape[2] == 0);
  assert(stride.shape[1] == dim.shape[0] + 2 * offset.shape[0]);   // stride is the packed stride of the padded dims
  GPUConn conn = ctx->conn();
  a.dptr_ = ctx->arena().alloc(a.padded_elems() * a.elem_size());
  a.zero(conn);
  return a;
}
template <>
ad_tensor4 GPUBatchArray3D<float>::view_base() const {
  const Shape3D pd = padded_dim();
  const long long Wp = (long long)pd.shape[0], Hp = (long long)pd.shape[1], C = (long long)pd.shape[2];
  ad_tensor4 t;
  t.base = dptr_;
  t.N = (uint32_t)batch_; t.C = (uint32_t)C; t.H = (uint32_t)Hp; t.W = (uint32_t)Wp;
  if (storage_ == COMPUTE_F32_NCHW) { t.dtype = AD_F32; t.sn = C * Hp * Wp; t.sc = Hp * Wp; t.sy = Wp; t.sx = 1; }
  else { t.dtype = AD_BF16; t.sn = Hp * Wp * C; t.sc = 1; t.sy = Wp * C; t.sx = C; }
  return t;
}
template <>
ad_tensor4 GPUBatchArray3D<float>::view_interior() const {
  ad_tensor4 t = view_base();
  t.base = (char*)t.base + (offset_.shape[1] * t.sy + offset_.shape[0] * t.sx) * (long long)elem_size();
  t.H = (uint32_t)dim_.shape[1]; t.W = (uint32_t)dim_.shape[0];
  return t;
}
template <>
void* GPUBatchArray3D<float>::interior_dptr() const { return view_interior().base; }

template <>
void GPUBatchArray3D<float>::load_host_nchw(const float* src, GPUContext* ctx) const {
  const size_t n = dim_.flat_size() * batch_;
  GPUConn conn = ctx->conn();
  ctx->reserve_scratch(n * sizeof(float));
  float* tmp = (float*)ctx->get_scratch();
  CUDA_CHECK(cudaMemcpyAsync(tmp, src, n * sizeof(float), cudaMemcpyHostToDevice, conn.stream()));
  const long long W = dim_.shape[0], H = dim_.shape[1], C = dim_.shape[2];
  ad_tensor4 s = {tmp, AD_F32, (uint32_t)batch_, (uint32_t)C, (uint32_t)H, (uint32_t)W, C * H * W, H * W, W, 1};
  ad_tensor4 d = view_interior();
  AD_CHECK(ad_convert(&s, &d, 0, conn.stream()));
  conn.sync();
}
template <>
void GPUBatchArray3D<float>::load_host_nchw_rows(const float* src_full, size_t full_h, size_t row0, GPUContext* ctx) const {
  const size_t n = dim_.flat_size() * batch_;
  GPUConn conn = ctx->conn();
  ctx->reserve_scratch(n * sizeof(float));
  float* tmp = (float*)ctx->get_scratch();
  const long long W = dim_.shape[0], H = dim_.shape[1], C = dim_.shape[2];
  assert(row0 + (size_t)H <= full_h);
  CUDA_CHECK(cudaMemcpy2DAsync(tmp, (size_t)(H * W) * sizeof(float), src_full + row0 * (size_t)W, full_h * (size_t)W * sizeof(float),
                               (size_t)(H * W) * sizeof(float), (size_t)C * batch_, cudaMemcpyHostToDevice, conn.stream()));
  ad_tensor4 s = {tmp, AD_F32, (uint32_t)batch_, (uint32_t)C, (uint32_t)H, (uint32_t)W, C * H * W, H * W, W, 1};
  ad_tensor4 d = view_interior();
  AD_CHECK(ad_convert(&s, &d, 0, conn.stream()));
  conn.sync();
}
template <>
void GPUBatchArray3D<float>::load_host_nhwc_rows(const float* src_full, size_t full_h, size_t row0, float scale, GPUContext* ctx) const {
  const size_t n = dim_.flat_size() * batch_;
  GPUConn conn = ctx->conn();
  ctx->reserve_scratch(n * sizeof(float));
  float* tmp = (float*)ctx->get_scratch();
  const long long W = dim_.shape[0], H = dim_.shape[1], C = dim_.shape[2];
  assert(row0 + (size_t)H <= full_h);
  // one contiguous block of H*W*C floats per image
  CUDA_CHECK(cudaMemcpy2DAsync(tmp, (size_t)(H * W * C) * sizeof(float), src_full + row0 * (size_t)(W * C),
                               full_h * (size_t)(W * C) * sizeof(float), (size_t)(H * W * C) * sizeof(float), batch_,
                               cudaMemcpyHostToDevice, conn.stream()));
  if (scale != 1.0f) AD_CHECK(ad_array_scale(n, scale, tmp, tmp, conn.stream()));
  ad_tensor4 s = {tmp, AD_F32, (uint32_t)batch_, (uint32_t)C, (uint32_t)H, (uint32_t)W, H * W * C, 1, W * C, C};
  ad_tensor4 d = view_interior();
  AD_CHECK(ad_convert(&s, &d, 0, conn.stream()));
  conn.sync();
}
template <>
void GPUBatchArray3D<float>::store_host_nchw(float* dst, GPUContext* ctx) const {
  const size_t n = dim_.flat_size() * batch_;
  GPUConn conn = ctx->conn();
  ctx->reserve_scratch(n * sizeof(float));
  float* tmp = (float*)ctx->get_scratch();
  const long long W = dim_.shape[0], H = dim_.shape[1], C = dim_.shape[2];
  ad_tensor4 d = {tmp, AD_F32, (uint32_t)batch_, (uint32_t)C, (uint32_t)H, (uint32_t)W, C * H * W, H * W, W, 1};
  ad_tensor4 s = view_interior();
  AD_CHECK(ad_convert(&s, &d, 0, conn.stream()));
  CUDA_CHECK(cudaMemcpyAsync(dst, tmp, n * sizeof(float), cudaMemcpyDeviceToHost, conn.stream()));
  conn.sync();
}

// ------------------------------------------------------------------ identity counters (thread-local, as the reference)
static thread_local uint64_t g_node = 0, g_epoch = 0, g_txn = 0, g_var = 0;
NodeId::NodeId() : id_(++g_node) {}
EpochId::EpochId() : id_(++g_epoch) {}
TxnId::TxnId() : id_(++g_txn) {}
VarId::VarId() : id_(++g_var), kind_(VAR_KIND_VAL) {}
VarId::VarId(VarKind k) : id_(++g_var), kind_(k) {}

// ------------------------------------------------------------------ graph walk
size_t OperatorStack::push(EpochId e) {
  if (entries_.empty() || entries_.back().epoch != e.raw_id()) entries_.push_back(Entry{e.raw_id(), 0, 0});
  return ++entries_.back().push_count;
}
size_t OperatorStack::degree(EpochId e) {
  assert(!entries_.empty() && entries_.back().epoch == e.raw_id());
  return entries_.back().push_count;
}
size_t OperatorStack::pop(EpochId e) {
  assert(!entries_.empty() && entries_.back().epoch == e.raw_id());
  size_t n = ++entries_.back().pop_count;
  if (n == entries_.back().push_count) entries_.pop_back();
  return n;
}

void Op::_push(EpochId epoch, function<void(Op*)> apply) {
  if (1 == stack_.push(epoch)) {
    for (auto& in : inputs_) in->_push(epoch, apply);
    apply(this);
  }
}
void Op::_pop(EpochId epoch, function<void(Op*)> apply) {
  if (stack_.degree(epoch) == stack_.pop(epoch)) {
    apply(this);
    for (auto it = inputs_.rbegin(); it != inputs_.rend(); ++it) (*it)->_pop(epoch, apply);
  }
}

static void walk_pop(Op* root, function<void(Op*)> apply) {
  EpochId e;
  root->_push(e, [](Op*) {});
  root->_pop(e, apply);
}
// Flat layouts.  The reference lays variables out in the pop order of the walk (op.hh:831-861) and
// relies on every rank's sub-graph giving the same order.  With operators shared between ranks the
// pop order of one rank's variables depends on where the walk enters, so here the operators that the
// walk reaches are visited in CREATION order (NodeIds increase monotonically): builders create the
// same layers in the same order on every rank, hence identical layouts on every rank.
template <typename F>
static size_t ordered_io(Op* root, VarIdSet& vars, size_t offset, F call) {
  vector<Op*> ops;
  walk_pop(root, [&](Op* op) { ops.push_back(op); });
  std::sort(ops.begin(), ops.end(), [](Op* a, Op* b) { return a->id().raw_id() < b->id().raw_id(); });
  vars.lock();
  for (Op* op : ops) offset = call(op, offset);
  vars.unlock();
  return offset;
}
size_t Op::load_val(TxnId txn, VarIdSet& vars, size_t offset, any* reader) {
  return ordered_io(this, vars, offset, [&](Op* op, size_t off) { return op->_load_val(txn, vars, off, reader); });
}
size_t Op::load_grad(TxnId txn, VarIdSet& vars, size_t offset, any* reader) {
  return ordered_io(this, vars, offset, [&](Op* op, size_t off) { return op->_load_grad(txn, vars, off, reader); });
}
size_t Op::store_val(TxnId txn, VarIdSet& vars, size_t offset, any* writer) {
  return ordered_io(this, vars, offset, [&](Op* op, size_t off) { return op->_store_val(txn, vars, off, writer); });
}
size_t Op::store_grad(TxnId txn, VarIdSet& vars, size_t offset, any* writer) {
  return ordered_io(this, vars, offset, [&](Op* op, size_t off) { return op->_store_grad(txn, vars, off, writer); });
}
void Op::init(TxnId txn, std::mt19937_64* rng) {
  EpochId e;
  _push(e, [&](Op* op) { op->_init(txn, rng); });
  _pop(e, [](Op*) {});
}
void Op::persist(TxnId txn, VarIdSet& vars) {
  EpochId e;
  _push(e, [&](Op* op) { op->_persist(txn, vars); });
  _pop(e, [](Op*) {});
}
void Op::eval(TxnId txn) {
  EpochId e;
  _push(e, [&](Op* op) { op->_forward(txn); });
  _pop(e, [](Op*) {});
}
void Op::backward(TxnId txn) {
  EpochId e;
  _push(e, [](Op*) {});
  _pop(e, [&](Op* op) { op->_backward(txn); });
  GPUContext::JoinAllSides();   // filter gradients issued on side streams are complete for whatever follows
}
void Op::gradient(TxnId txn) {
  eval(txn);
  _set_grad_sink(txn);
  backward(txn);
}

}  // namespace arraydiff
