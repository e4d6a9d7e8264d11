// Schedules and the parallel SGD optimizer.  Same configuration and update rule as the reference's
// include/arraydiff/optimize.hh (schedules :19-125, SGDConfig :127-136, ParallelSGDOptimizer :262-586;
// update :479-499).  What differs is the data movement: the reference reduces all gradients to rank 0,
// updates there and broadcasts the parameters (two hops, root-only arithmetic, full device syncs);
// here the flat gradient buffer is all-reduced (NVLink / NCCL) and every rank applies the same fused
// update kernel to its own replica, so no broadcast is needed.
#ifndef ARRAYDIFF_OPTIMIZE_HH
#define ARRAYDIFF_OPTIMIZE_HH

#include <map>
#include <utility>

#include "arraydiff/op.hh"

namespace arraydiff {

template <typename T>
class Schedule {
public:
  virtual ~Schedule() {}
  virtual T at(size_t iteration) = 0;
};
template <typename T>
class ConstantSchedule : public Schedule<T> {
public:
  explicit ConstantSchedule(T v) : v_(v) {}
  T at(size_t) override { return v_; }
private:
  T v_;
};
// `init` until the first step, then each value from its step on: PiecewiseStepSchedule(0.1, 150000, 0.01, 300000, 0.001)
// (the argument forms of the reference, include/arraydiff/optimize.hh:44-90), or a map {step: value}.
template <typename T>
class PiecewiseStepSchedule : public Schedule<T> {
public:
  explicit PiecewiseStepSchedule(T init) : init_(init) {}
  PiecewiseStepSchedule(T init, std::map<size_t, T> steps) : init_(init), steps_(steps) {}
  PiecewiseStepSchedule(T init, vector<std::pair<size_t, T>> pieces) : init_(init) { for (auto& p : pieces) steps_[p.first] = p.second; }
  template <typename... Rest>
  PiecewiseStepSchedule(T init, size_t step1, T val1, Rest... rest) : init_(init) { add(step1, val1, rest...); }
  T at(size_t it) override {
    T v = init_;
    for (auto& kv : steps_) if (it >= kv.first) v = kv.second;
    return v;
  }
private:
  void add() {}
  template <typename... Rest> void add(size_t step, T val, Rest... rest) { steps_[step] = val; add(rest...); }
  T init_;
  std::map<size_t, T> steps_;
};
// linear from `init` at step 0 to `val1` at `step1`, constant afterwards (reference :92-130)
template <typename T>
class PiecewiseLinearSchedule : public Schedule<T> {
public:
  explicit PiecewiseLinearSchedule(T init) : init_(init), step1_(0), val1_(init) {}
  PiecewiseLinearSchedule(T init, size_t step1, T val1) : init_(init), step1_(step1), val1_(val1) {}
  T at(size_t it) override {
    if (step1_ == 0 || it >= step1_) return val1_;
    return init_ + (val1_ - init_) * (T)it / (T)step1_;
  }
private:
  T init_;
  size_t step1_;
  T val1_;
};

class SGDConfig {
public:
  size_t minibatch_size = 1;
  size_t compute_batch_size = 1;
  shared_ptr<Schedule<double>> step_size;
  shared_ptr<Schedule<double>> momentum;
  bool nesterov = false;
  double l2_reg = 0.0;
  double batch_norm_rate = 0.0;
};

template <typename T>
class ParallelSGDOptimizer {
public:
  // `sink` joins every rank's sub-graph; params / grads are the per-rank variable sets.
  ParallelSGDOptimizer(SGDConfig cfg, shared_ptr<Op> sink, vector<VarIdSet> params, vector<VarIdSet> grads)
      : cfg_(cfg), sink_(sink), params_(params), grads_(grads), param_dim_(0), iter_count_(0) {}
  // The reference's constructor (include/arraydiff/optimize.hh:265): batch_stats are the per-rank sets of the batch
  // normalisation layers' batch mean / variance variables, fixed_stats the matching running statistics.
  ParallelSGDOptimizer(SGDConfig cfg, shared_ptr<Op> sum_loss, vector<VarIdSet> params, vector<VarIdSet> grads,
                       vector<VarIdSet> batch_stats, vector<VarIdSet> fixed_stats)
      : cfg_(cfg), sink_(sum_loss), params_(params), grads_(grads), batch_stats_(batch_stats), fixed_stats_(fixed_stats),
        param_dim_(0), iter_count_(0) {}

  size_t param_dim() const { return param_dim_; }
  size_t iteration() const { return iter_count_; }
  // A replayed (graph-captured) step does its update on the device only: the host-side iteration
  // counter, which indexes the schedules, is advanced here.
  void skip_iterations(size_t n) { iter_count_ += n; }
  // the three schedule values the next step() bakes into its update kernel
  void schedule_now(float out[3]) const {
    out[0] = (float)cfg_.momentum->at(iter_count_);
    out[1] = (float)cfg_.step_size->at(iter_count_);
    out[2] = (float)cfg_.step_size->at(iter_count_ + 1);
  }

  // Draws the initial parameters, makes every rank's replica equal to rank 0's and sets up the flat
  // parameter / gradient / momentum buffers (reference :314-386).
  void reset(shared_ptr<Context> ctx, std::mt19937_64* rng);
  // The reference's form (:314-386): the graph was initialised by the caller (op->init); rank 0's parameters and
  // running statistics become every rank's, the flat buffers are set up.
  void reset(shared_ptr<Context> parallel_ctx);
  // The reference's training step (:389-564): ceil(minibatch / compute batch) micro-batches, each a fresh transaction
  // handed to `compute_batch_fn(txn, batch size, loss)` (which persists the parameters, loads data and calls
  // loss->gradient(txn)); gradients are summed over micro-batches, batch statistics averaged; then the gradient is
  // summed over ranks, L2 + (Nesterov) momentum SGD is applied, the running statistics move towards the step's
  // average batch statistics by batch_norm_rate, and parameters / statistics are loaded back into the graph.
  // Differs from the reference in the data movement only: all-reduce and update on every rank instead of
  // reduce -> update on rank 0 -> broadcast.
  void step(function<void(TxnId, size_t, shared_ptr<Op>)>& compute_batch_fn, shared_ptr<Context> parallel_ctx);
  void step(function<void(TxnId, size_t, shared_ptr<Op>)>&& compute_batch_fn, shared_ptr<Context> parallel_ctx) {
    step(compute_batch_fn, parallel_ctx);
  }
  size_t stat_dim() const { return stat_dim_; }
  void store_fixed_stats(size_t rank, float* host);
  // Flat-parameter checkpoint: the flat buffers the graph walk fills (parameters in store_val order, the momentum
  // buffer, the running statistics; reference include/arraydiff/optimize.hh:146-165, :228-238 keeps exactly these
  // as its optimizer state) written to one file with a header that names every variable:
  //   "ADB2CKPT" | u32 version = 1 | u64 param_dim | u64 stat_dim | u64 iteration | u32 entries |
  //   entries x { u32 name length | name bytes | u64 offset | u64 size } | fp32 params[param_dim] |
  //   fp32 momentum[param_dim] | fp32 running statistics[stat_dim]          (little endian, no padding)
  // save: the first local rank's copy (all replicas are identical).  load: checks the dimensions and the manifest,
  // then gives every local rank the file's state (buffers, graph variables, iteration counter).  Both synchronise.
  bool save_checkpoint(const string& path);
  bool load_checkpoint(const string& path);
  // Worker 0's parameters and running statistics become every process's (a context made with MakeDistributed, with
  // or without set_world): the others contribute zeros to one sum over the gradient exchange, so the bits are worker
  // 0's.  The broadcast-init of the reference's multi-process optimizer (include/arraydiff/optimize_mpi.hh:66-95).
  void broadcast_from_worker0();
  // To be called after the gradients of transaction `txn` exist on every rank: gathers them into the
  // flat buffer, sums over ranks, applies L2 + (Nesterov) momentum SGD on every rank, and loads the
  // new parameters back into the graph (reference :407-561).
  void step(TxnId txn);
  // carries parameters into a new transaction (to be called before each forward pass)
  void persist(TxnId txn);
  // flat fp32 views for tests / checkpoints
  void store_params(size_t rank, float* host);
  void load_params(const float* host);
  void store_sum_grads(size_t rank, float* host);

private:
  SGDConfig cfg_;
  shared_ptr<Op> sink_;
  vector<VarIdSet> params_, grads_, batch_stats_, fixed_stats_;
  size_t param_dim_, iter_count_, stat_dim_ = 0;
  vector<GPUMemory<T>> batch_grad_, batch_stat_, avg_stat_, running_stat_;
  MultiGPUContext* mgpu_ = nullptr;
  shared_ptr<Context> ctx_;
  vector<GPUMemory<T>> param_, sum_grad_, momentum_;
};

// Data-parallel SGD over processes, one replica of the (possibly spatially partitioned) net per process: the
// reference's MPIDataParallelSGDOptimizer (include/arraydiff/optimize_mpi.hh:20-205) with the built-in peer exchange
// of MultiGPUContext (or an NCCL hook) in place of MPI_Bcast / MPI_Allreduce.  reset() makes worker 0's initial point
// everyone's; step() sums the gradients of all workers (no averaging, as the reference) and applies the same update
// everywhere.  The context must be one made with MultiGPUContext::MakeDistributed whose peers (set_peer_arena /
// set_world_peer_arena) are the other workers.
template <typename T>
class DataParallelSGDOptimizer {
public:
  DataParallelSGDOptimizer(SGDConfig cfg, shared_ptr<Op> sum_loss, VarIdSet params, VarIdSet grads, VarIdSet batch_stats,
                           VarIdSet fixed_stats)
      : cfg_(cfg), sum_loss_(sum_loss), params_(params), grads_(grads), batch_stats_(batch_stats), fixed_stats_(fixed_stats) {}
  size_t worker_rank() const { return worker_rank_; }
  size_t num_workers() const { return num_workers_; }
  void reset(shared_ptr<Context> ctx) {
    auto* m = dynamic_cast<MultiGPUContext*>(ctx.get());
    assert(m && m->distributed());
    worker_rank_ = m->exchange_rank(); num_workers_ = m->exchange_size();
    vector<VarIdSet> p(m->num_ranks()), g(m->num_ranks()), b(m->num_ranks()), f(m->num_ranks());
    p[m->my_rank()] = params_; g[m->my_rank()] = grads_; b[m->my_rank()] = batch_stats_; f[m->my_rank()] = fixed_stats_;
    inner_.reset(new ParallelSGDOptimizer<T>(cfg_, sum_loss_, p, g, b, f));
    inner_->reset(ctx);
    inner_->broadcast_from_worker0();
  }
  void step(function<void(TxnId, size_t, shared_ptr<Op>)>& compute_batch_fn, shared_ptr<Context> ctx) { inner_->step(compute_batch_fn, ctx); }
  ParallelSGDOptimizer<T>& inner() { return *inner_; }
private:
  SGDConfig cfg_;
  shared_ptr<Op> sum_loss_;
  VarIdSet params_, grads_, batch_stats_, fixed_stats_;
  size_t worker_rank_ = 0, num_workers_ = 1;
  std::unique_ptr<ParallelSGDOptimizer<T>> inner_;
};

}  // namespace arraydiff
#endif
