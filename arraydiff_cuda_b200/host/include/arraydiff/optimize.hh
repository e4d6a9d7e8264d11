// Schedules and the parallel SGD optimizer.  Same configuration and update rule as the reference's
// include/arraydiff/optimize.hh (schedules :19-125, SGDConfig :127-136, ParallelSGDOptimizer :262-586;
// update :479-499).  What differs is the data movement: the reference reduces all gradients to rank 0,
// updates there and broadcasts the parameters (two hops, root-only arithmetic, full device syncs);
// here the flat gradient buffer is all-reduced (NVLink / NCCL) and every rank applies the same fused
// update kernel to its own replica, so no broadcast is needed.
#ifndef ARRAYDIFF_OPTIMIZE_HH
#define ARRAYDIFF_OPTIMIZE_HH

#include <map>

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
// value changes at the given iterations: {0: a, 1000: b, ...}
template <typename T>
class PiecewiseStepSchedule : public Schedule<T> {
public:
  PiecewiseStepSchedule(T init, std::map<size_t, T> steps) : init_(init), steps_(steps) {}
  T at(size_t it) override {
    T v = init_;
    for (auto& kv : steps_) if (it >= kv.first) v = kv.second;
    return v;
  }
private:
  T init_;
  std::map<size_t, T> steps_;
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
  vector<VarIdSet> params_, grads_;
  size_t param_dim_, iter_count_;
  MultiGPUContext* mgpu_ = nullptr;
  shared_ptr<Context> ctx_;
  vector<GPUMemory<T>> param_, sum_grad_, momentum_;
};

}  // namespace arraydiff
#endif
