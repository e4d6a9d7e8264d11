// C entry points over the C++ host layer, for drivers that are not C++ (the Python tests and the
// benchmark): build a context and a net, feed host tensors, run forward / backward / update, read
// results back.  Handles are opaque pointers; functions return 0 or a negative ad_status.
#include <cstring>
#include <memory>
#include <vector>

#include "arraydiff/optimize.hh"
#include "arraydiff/zoo.hh"

using namespace arraydiff;

namespace {
struct Net {
  shared_ptr<MultiGPUContext> ctx;
  SpatialParallelNet net;
  ConvNetConfig cfg;
  std::unique_ptr<ParallelSGDOptimizer<float>> opt;
  std::unique_ptr<TxnId> txn;
  std::mt19937_64 rng;
  // the resident step captured as one CUDA graph (adh_net_step_graph)
  cudaGraphExec_t gexec = nullptr;
  int g_update = 0;
  float g_key[3] = {0.f, 0.f, 0.f};
  uint64_t g_launches = 0;
};
struct Ctx { shared_ptr<MultiGPUContext> ctx; };
}  // namespace

extern "C" {

void* adh_context_create(const int* devices, int n, int mode, size_t arena_mb) {
  vector<int> devs(devices, devices + n);
  auto* c = new Ctx{MultiGPUContext::Make(devs, (ComputeMode)mode, arena_mb << 20)};
  return c;
}
void* adh_context_create_distributed(int rank, int world, int device, int mode, size_t arena_mb) {
  return new Ctx{MultiGPUContext::MakeDistributed((size_t)rank, (size_t)world, device, (ComputeMode)mode, arena_mb << 20)};
}
void adh_context_destroy(void* c) { delete (Ctx*)c; }
int adh_context_arena_handle(void* c, uint8_t out[64]) {
  auto& m = ((Ctx*)c)->ctx;
  return ad_ipc_get_handle(m->arena_base(m->my_rank()), out);
}
int adh_context_set_peer_handle(void* c, int rank, const uint8_t handle[64]) {
  auto& m = ((Ctx*)c)->ctx;
  void* p = nullptr;
  GPUConn conn = m->device_context(m->my_rank())->conn();
  int st = ad_ipc_open_handle(handle, &p);
  if (st != AD_OK) return st;
  m->set_peer_arena((size_t)rank, p);
  return AD_OK;
}
// data-parallel replicas around the spatial group: this process is world_rank of world_size (see
// MultiGPUContext::set_world); then one call per other process with its arena's IPC handle
int adh_context_set_world(void* c, int world_rank, int world_size) {
  if (world_rank < 0 || world_size <= 0 || world_rank >= world_size || world_size > ARRAYDIFF_MAX_PEERS) return AD_ERR_BAD_ARG;
  ((Ctx*)c)->ctx->set_world((size_t)world_rank, (size_t)world_size);
  return AD_OK;
}
int adh_context_set_world_peer_handle(void* c, int world_rank, const uint8_t handle[64]) {
  auto& m = ((Ctx*)c)->ctx;
  void* p = nullptr;
  GPUConn conn = m->device_context(m->my_rank())->conn();
  int st = ad_ipc_open_handle(handle, &p);
  if (st != AD_OK) return st;
  m->set_world_peer_arena((size_t)world_rank, p);
  return AD_OK;
}
// a world peer that is also a member of this process's spatial group: reuse the mapping made for the group
// (an IPC handle is opened once per process)
int adh_context_set_world_peer_from_group(void* c, int world_rank, int group_rank) {
  auto& m = ((Ctx*)c)->ctx;
  if (group_rank < 0 || (size_t)group_rank >= m->num_ranks() || !m->arena_base((size_t)group_rank)) return AD_ERR_BAD_ARG;
  m->set_world_peer_arena((size_t)world_rank, m->arena_base((size_t)group_rank));
  return AD_OK;
}
void adh_context_set_allreduce_hook(void* c, void (*fn)(float*, size_t, cudaStream_t, void*), void* user) {
  ((Ctx*)c)->ctx->set_allreduce_hook(fn, user);
}
// One halo exchange (op 0) or accumulate-back (op 1) through Spatial2DComm on a grid_h x grid_w grid laid over the
// context's ranks (one process): bufs[r] is rank r's padded device buffer.  Runs the reference's call sequence --
// group_start, halo_exchange / halo_reduce, group_end on every rank (src/op.cc:2977-3000) -- with a communicator array
// made by Spatial2DComm::InitAll(comms, grid_w, grid_h).
int adh_context_halo2d(void* c, int grid_w, int grid_h, int op, int nhwc, int bf16, uint32_t p, uint32_t w, uint32_t h, uint32_t ch,
                       uint32_t n, void** bufs) {
  auto& m = ((Ctx*)c)->ctx;
  if (m->distributed() || (size_t)(grid_w * grid_h) != m->num_ranks()) return AD_ERR_BAD_ARG;
  std::vector<Spatial2DComm> comms(m->num_ranks());
  Spatial2DComm::InitAll(comms.data(), (uint32_t)grid_w, (uint32_t)grid_h, m.get());
  const auto fmt = nhwc ? SPATIAL2D_TENSOR_NHWC : SPATIAL2D_TENSOR_NCHW;
  const auto dt = bf16 ? SPATIAL2D_DATA_BFLOAT16 : SPATIAL2D_DATA_FLOAT;
  for (size_t r = 0; r < m->num_ranks(); ++r) comms[r].group_start();
  for (size_t r = 0; r < m->num_ranks(); ++r) {
    if (op == 0) comms[r].halo_exchange(bufs[r], p, w, h, ch, n, fmt, dt);
    else comms[r].halo_reduce(bufs[r], p, w, h, ch, n, fmt, dt);
  }
  for (size_t r = 0; r < m->num_ranks(); ++r) {
    GPUConn conn = m->device_context(r)->conn();
    comms[r].group_end(conn);
  }
  m->sync();
  return AD_OK;
}
void* adh_context_stream(void* c, int rank) { return (void*)((Ctx*)c)->ctx->device_context((size_t)rank)->stream(); }

// kind: "conv3x3" (filters = output channels) or "stem_stage1"
void* adh_net_create(void* c, const char* kind, int H, int W, int C, int batch, int filters, uint64_t seed) {
  auto* n = new Net();
  n->ctx = ((Ctx*)c)->ctx;
  n->cfg.input_h = (size_t)H; n->cfg.input_w = (size_t)W; n->cfg.input_c = (size_t)C; n->cfg.batch_size = (size_t)batch;
  n->rng.seed(seed);
  if (!std::strcmp(kind, "conv3x3")) n->net = SpatialParallelResNet<float>::MakeConv3x3(n->cfg, (size_t)filters, n->ctx);
  else if (!std::strcmp(kind, "conv3x3_repad")) n->net = SpatialParallelResNet<float>::MakeConv3x3(n->cfg, (size_t)filters, n->ctx, 3);
  else if (!std::strcmp(kind, "conv3x3_collectives")) n->net = SpatialParallelResNet<float>::MakeConv3x3Collectives(n->cfg, (size_t)filters, n->ctx);
  else if (!std::strcmp(kind, "stem_stage1")) n->net = SpatialParallelResNet<float>::MakeStemStage1(n->cfg, n->ctx);
  else if (!std::strcmp(kind, "parallel_resnet18")) n->net = SpatialParallelResNet<float>::MakeParallelResNet18(n->cfg, filters > 0 ? (size_t)filters : 1000, n->ctx);
  else if (!std::strcmp(kind, "parallel_resnet50")) n->net = SpatialParallelResNet<float>::MakeParallelResNet50(n->cfg, filters > 0 ? (size_t)filters : 1000, n->ctx);
  else if (!std::strncmp(kind, "segnet", 6)) {
    // "segnet50": ResNet-50 depth; "segnet_small": one block per stage; `filters` (if > 0) = stem width
    SegNetConfig seg;
    if (filters > 0) seg.base = (size_t)filters;
    if (!std::strcmp(kind, "segnet_small")) for (auto& b : seg.blocks) b = 1;
    else if (std::strcmp(kind, "segnet50")) { delete n; return nullptr; }
    n->net = SpatialParallelResNet<float>::MakeSegNet50(n->cfg, seg, n->ctx);
  }
  else { delete n; return nullptr; }
  SGDConfig sc;
  sc.step_size = make_shared<ConstantSchedule<double>>(0.1);
  sc.momentum = make_shared<ConstantSchedule<double>>(0.9);
  n->opt.reset(new ParallelSGDOptimizer<float>(sc, n->net.sink, n->net.dev_params, n->net.dev_grads));
  n->opt->reset(n->ctx, &n->rng);
  return n;
}
void adh_net_destroy(void* h) { delete (Net*)h; }
// flat-parameter checkpoint of the net's optimizer state (parameters, momentum, running statistics, iteration)
int adh_net_save_checkpoint(void* h, const char* path) { return ((Net*)h)->opt->save_checkpoint(path) ? AD_OK : AD_ERR_BAD_ARG; }
int adh_net_load_checkpoint(void* h, const char* path) {
  auto* n = (Net*)h;
  if (!n->opt->load_checkpoint(path)) return AD_ERR_BAD_ARG;
  if (n->gexec) { cudaGraphExecDestroy(n->gexec); n->gexec = nullptr; }   // schedule values may differ: record again
  return AD_OK;
}
// worker 0's parameters become every process's (contexts made with adh_context_create_distributed)
int adh_net_broadcast_params(void* h) { ((Net*)h)->opt->broadcast_from_worker0(); return AD_OK; }
size_t adh_net_iteration(void* h) { return ((Net*)h)->opt->iteration(); }
int adh_net_configure_sgd(void* h, double step_size, double momentum, double l2, int nesterov) {
  auto* n = (Net*)h;
  SGDConfig sc;
  sc.step_size = make_shared<ConstantSchedule<double>>(step_size);
  sc.momentum = make_shared<ConstantSchedule<double>>(momentum);
  sc.l2_reg = l2; sc.nesterov = nesterov != 0;
  vector<float> keep(n->opt->param_dim());
  size_t first = n->ctx->distributed() ? n->ctx->my_rank() : 0;
  n->opt->store_params(first, keep.data());
  n->opt.reset(new ParallelSGDOptimizer<float>(sc, n->net.sink, n->net.dev_params, n->net.dev_grads));
  std::mt19937_64 rng(1);
  n->opt->reset(n->ctx, &rng);
  n->opt->load_params(keep.data());
  return AD_OK;
}
// "name offset size\n" per parameter of the flat buffer (rank 0's order; every rank's is the same)
size_t adh_net_param_manifest(void* h, char* buf, size_t cap) {
  auto* n = (Net*)h;
  size_t first = n->ctx->distributed() ? n->ctx->my_rank() : 0;
  ParamManifest m;
  any w = &m;
  TxnId t;
  n->net.sink->store_val(t, n->net.dev_params[first], 0, &w);
  string out;
  for (auto& e : m) out += e.name + " " + std::to_string(e.offset) + " " + std::to_string(e.size) + "\n";
  if (buf && cap) { std::strncpy(buf, out.c_str(), cap - 1); buf[cap - 1] = 0; }
  return out.size();
}
size_t adh_net_param_count(void* h) { return ((Net*)h)->opt->param_dim(); }
int adh_net_get_params(void* h, int rank, float* host) { ((Net*)h)->opt->store_params((size_t)rank, host); return AD_OK; }
int adh_net_set_params(void* h, const float* host) { ((Net*)h)->opt->load_params(host); return AD_OK; }
// dims of one rank's output strip: N, C, h, W
void adh_net_output_dims(void* h, int dims[4]) {
  auto* n = (Net*)h;
  ActVar o;
  for (auto& x : n->net.outputs) if (x) { o = x; break; }
  Shape3D d = o->shape();
  dims[0] = (int)o->batch_shape(); dims[1] = (int)d.shape[2]; dims[2] = (int)d.shape[1]; dims[3] = (int)d.shape[0];
}
// full image, packed NCHW fp32 on the host; starts a new transaction and runs the forward pass
// host image (packed NCHW fp32) -> the input variable of every local rank (its H-strip, or the whole image), in a new
// transaction; nothing is evaluated.  adh_net_step_resident / adh_net_step_graph then run on what was loaded.
int adh_net_load_input(void* h, const float* image_nchw) {
  auto* n = (Net*)h;
  n->txn.reset(new TxnId());
  n->opt->persist(*n->txn);
  for (auto& in : n->net.inputs) {
    if (!in) continue;
    VarIdSet v = VarIdSet::Singleton(in->data().val.var());
    const size_t h = in->shape().shape[1];
    any rd;
    if (h != n->cfg.input_h) rd = HostRows{image_nchw, n->cfg.input_h, in->rank() * h};   // the rank's strip, straight from the host image
    else rd = const_cast<float*>(image_nchw);                                             // the whole image on every rank
    n->net.sink->load_val(*n->txn, v, 0, &rd);
  }
  return AD_OK;
}
int adh_net_forward(void* h, const float* image_nchw) {
  auto* n = (Net*)h;
  adh_net_load_input(h, image_nchw);
  n->net.sink->eval(*n->txn);
  n->ctx->end_phase();
  return AD_OK;
}
int adh_net_get_output(void* h, int rank, float* host_strip) {
  auto* n = (Net*)h;
  for (auto& o : n->net.outputs) {
    if ((int)o->rank() != rank) continue;
    VarIdSet v = VarIdSet::Singleton(o->data().val.var());
    any w = host_strip;
    n->net.sink->store_val(*n->txn, v, 0, &w);
    return AD_OK;
  }
  return AD_ERR_BAD_ARG;
}
int adh_net_set_output_grad(void* h, int rank, const float* host_strip) {
  auto* n = (Net*)h;
  for (auto& o : n->net.outputs) {
    if ((int)o->rank() != rank) continue;
    any rd = const_cast<float*>(host_strip);
    n->net.sink->load_grad(*n->txn, n->net.output_grad_vars[(size_t)rank], 0, &rd);
    return AD_OK;
  }
  return AD_ERR_BAD_ARG;
}
int adh_net_backward(void* h) {
  auto* n = (Net*)h;
  n->net.sink->backward(*n->txn);
  n->ctx->end_phase();
  return AD_OK;
}
// flat gradient of rank's parameters (this rank's strip only, before the allreduce)
int adh_net_get_param_grads(void* h, int rank, float* host) {
  auto* n = (Net*)h;
  GPUContext* g = n->ctx->device_context((size_t)rank).get();
  GPUMemory<float> tmp(n->opt->param_dim(), g);
  any w = tmp;
  n->net.sink->store_grad(*n->txn, n->net.dev_grads[(size_t)rank], 0, &w);
  GPUConn conn = g->conn();
  tmp.store_sync(host, n->opt->param_dim(), 0, conn);
  return AD_OK;
}
// gradient w.r.t. the full image as seen by `rank` (non-zero only on its rows)
int adh_net_get_input_grad(void* h, int rank, float* host_full) {
  auto* n = (Net*)h;
  auto& in = n->net.inputs[(size_t)rank];
  if (!in) return AD_ERR_BAD_ARG;
  VarIdSet v = VarIdSet::Singleton(in->data().grad.var());
  any w = host_full;
  n->net.sink->store_grad(*n->txn, v, 0, &w);
  return AD_OK;
}
// One full step on data that is already resident on the device: the image loaded by the last
// adh_net_forward and the output gradients loaded by the last adh_net_set_output_grad are carried into a
// new transaction; forward, backward and (optionally) gradient allreduce + SGD update run without any
// host transfer or synchronisation.
int adh_net_step_resident(void* h, int with_update) {
  auto* n = (Net*)h;
  n->txn.reset(new TxnId());
  n->opt->persist(*n->txn);
  n->net.sink->persist(*n->txn, n->net.input_vars);
  n->net.sink->eval(*n->txn);
  if (n->net.losses.empty())   // a net that ends in a loss makes its own output gradient
    for (size_t r = 0; r < n->ctx->num_ranks(); ++r)
      if (n->ctx->is_local(r)) n->net.sink->load_grad(*n->txn, n->net.output_grad_vars[r], 0, nullptr);
  n->net.sink->backward(*n->txn);
  if (with_update) n->opt->step(*n->txn);
  n->ctx->end_phase();
  return AD_OK;
}
// labels of `rank`'s strip, uint32 [N][h][W] (nets that end in the per-pixel loss)
int adh_net_set_labels(void* h, int rank, const uint32_t* host) {
  auto* n = (Net*)h;
  for (auto& l : n->net.losses)
    if ((int)l->rank() == rank) { l->load_labels(host); return AD_OK; }
  return AD_ERR_BAD_ARG;
}
// weight of every per-pixel (per-image) loss term in the gradient, e.g. 1 / (global batch x ranks per replica group)
// when several data-parallel groups sum their gradients
int adh_net_set_loss_weight(void* h, float w) {
  auto* n = (Net*)h;
  if (n->net.losses.empty()) return AD_ERR_BAD_ARG;
  for (auto& l : n->net.losses) l->set_loss_weight(w);
  return AD_OK;
}
// sum of the per-pixel losses of the local ranks' strips and the number of pixels behind it (synchronous)
int adh_net_loss(void* h, double* sum, uint64_t* pixels) {
  auto* n = (Net*)h;
  if (n->net.losses.empty()) return AD_ERR_BAD_ARG;
  double s = 0.0;
  uint64_t px = 0;
  for (auto& l : n->net.losses) { s += l->loss_sum(); px += l->pixels(); }
  *sum = s; *pixels = px;
  return AD_OK;
}
// gradient of an output strip (packed NCHW fp32): what the loss wrote, or what set_output_grad loaded
int adh_net_get_output_grad(void* h, int rank, float* host_strip) {
  auto* n = (Net*)h;
  for (auto& o : n->net.outputs) {
    if ((int)o->rank() != rank) continue;
    VarIdSet v = VarIdSet::Singleton(o->data().grad.var());
    any w = host_strip;
    n->net.sink->store_grad(*n->txn, v, 0, &w);
    return AD_OK;
  }
  return AD_ERR_BAD_ARG;
}
// The same step replayed from a CUDA graph.  The first call (and any call after the schedule values or
// `with_update` changed) records adh_net_step_resident on the ranks' streams -- rank 0's stream is the
// origin, the other local ranks' streams are forked from it and joined back -- and instantiates the
// graph; every call launches it once.  Buffers are arena-resident, so addresses are stable between
// steps.  One process per GPU keeps the eager path: its flag epochs change every step.
int adh_net_step_graph(void* h, int with_update) {
  auto* n = (Net*)h;
  // one process per GPU: replayable when the gradient allreduce is the built-in peer exchange (a hook may
  // call into a library that cannot be captured)
  if (n->ctx->distributed() && n->ctx->has_allreduce_hook()) return adh_net_step_resident(h, with_update);
  float key[3];
  n->opt->schedule_now(key);
  if (n->gexec && (n->g_update != with_update || std::memcmp(key, n->g_key, sizeof key))) {
    cudaGraphExecDestroy(n->gexec);
    n->gexec = nullptr;
  }
  const bool dist = n->ctx->distributed();
  const size_t R = dist ? 1 : n->ctx->num_ranks(), first = dist ? n->ctx->my_rank() : 0;
  cudaStream_t origin = n->ctx->device_context(first)->stream();
  if (!n->gexec) {
    GPUConn c0 = n->ctx->device_context(first)->conn();
    CUDA_CHECK(cudaStreamBeginCapture(origin, cudaStreamCaptureModeRelaxed));
    vector<cudaEvent_t> evs;
    cudaEvent_t fork;
    CUDA_CHECK(cudaEventCreateWithFlags(&fork, cudaEventDisableTiming));
    CUDA_CHECK(cudaEventRecord(fork, origin));
    evs.push_back(fork);
    for (size_t r = 1; r < R; ++r) CUDA_CHECK(cudaStreamWaitEvent(n->ctx->device_context(r)->stream(), fork, 0));
    const uint64_t l0 = ad_launch_count();
    adh_net_step_resident(h, with_update);
    n->g_launches = ad_launch_count() - l0;
    for (size_t r = 1; r < R; ++r) {
      GPUConn cr = n->ctx->device_context(r)->conn();
      cudaEvent_t e;
      CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
      CUDA_CHECK(cudaEventRecord(e, n->ctx->device_context(r)->stream()));
      CUDA_CHECK(cudaStreamWaitEvent(origin, e, 0));
      evs.push_back(e);
    }
    cudaGraph_t graph = nullptr;
    GPUConn c1 = n->ctx->device_context(first)->conn();
    CUDA_CHECK(cudaStreamEndCapture(origin, &graph));
    CUDA_CHECK(cudaGraphInstantiate(&n->gexec, graph, 0));
    cudaGraphDestroy(graph);
    for (auto e : evs) cudaEventDestroy(e);
    n->g_update = with_update;
    std::memcpy(n->g_key, key, sizeof key);
    CUDA_CHECK(cudaGraphLaunch(n->gexec, origin));   // the recording itself executed nothing
    return AD_OK;
  }
  GPUConn c0 = n->ctx->device_context(first)->conn();
  CUDA_CHECK(cudaGraphLaunch(n->gexec, origin));
  if (with_update) n->opt->skip_iterations(1);
  return AD_OK;
}
// kernels one replay of the graph launches (0 before the first adh_net_step_graph)
uint64_t adh_net_graph_launches(void* h) { return ((Net*)h)->g_launches; }
// allreduce of the gradients + SGD update on every rank
int adh_net_sgd_step(void* h) { auto* n = (Net*)h; n->opt->step(*n->txn); n->ctx->end_phase(); return AD_OK; }
int adh_net_sync(void* h) { ((Net*)h)->ctx->sync(); return AD_OK; }
int adh_net_status(void* h) {
  auto* n = (Net*)h;
  int st = 0;
  for (size_t r = 0; r < n->ctx->num_ranks(); ++r) if (n->ctx->is_local(r)) { int s = n->ctx->device_context(r)->read_status(); if (s) st = s; }
  return st;
}
size_t adh_net_arena_used(void* h, int rank) { return ((Net*)h)->ctx->device_context((size_t)rank)->arena().used(); }

}  // extern "C"
