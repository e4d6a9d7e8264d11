#include "arraydiff/optimize.hh"

namespace arraydiff {

template <>
void ParallelSGDOptimizer<float>::persist(TxnId txn) {
  for (auto& p : params_) sink_->persist(txn, p);
}

template <>
void ParallelSGDOptimizer<float>::reset(shared_ptr<Context> ctx, std::mt19937_64* rng) {
  ctx_ = ctx;
  mgpu_ = dynamic_cast<MultiGPUContext*>(ctx.get());
  assert(mgpu_);
  const size_t R = mgpu_->num_ranks();
  TxnId init_txn;
  sink_->init(init_txn, rng);
  param_dim_ = 0;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    size_t d = sink_->store_val(init_txn, params_[r], 0, nullptr);
    assert(param_dim_ == 0 || param_dim_ == d);   // per-rank sub-graphs are built alike (reference :323-333)
    param_dim_ = d;
    assert(sink_->store_grad(init_txn, grads_[r], 0, nullptr) == d);
  }
  param_.resize(R); sum_grad_.resize(R); momentum_.resize(R);
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    GPUContext* g = mgpu_->device_context(r).get();
    param_[r] = GPUMemory<float>(param_dim_, g);
    sum_grad_[r] = GPUMemory<float>(param_dim_, g);
    momentum_[r] = GPUMemory<float>(param_dim_, g);
  }
  // rank 0's draw becomes everybody's initial point (reference :358-386).  Ranks in other processes
  // draw from an equally seeded generator and therefore hold the same values already.
  size_t first = mgpu_->distributed() ? mgpu_->my_rank() : 0;
  {
    any w = param_[first];
    sink_->store_val(init_txn, params_[first], 0, &w);
  }
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r) || r == first) continue;
    mgpu_->device_context(first)->sync();
    GPUConn conn = mgpu_->device_context(r)->conn();
    CUDA_CHECK(cudaMemcpyAsync(param_[r].dptr(), param_[first].dptr(), param_dim_ * 4, cudaMemcpyDeviceToDevice, conn.stream()));
  }
  TxnId load_txn;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    any rd = param_[r];
    sink_->load_val(load_txn, params_[r], 0, &rd);
  }
  iter_count_ = 0;
  mgpu_->sync();
}

template <>
void ParallelSGDOptimizer<float>::step(TxnId txn) {
  const size_t R = mgpu_->num_ranks();
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    any w = sum_grad_[r];
    sink_->store_grad(txn, grads_[r], 0, &w);
  }
  // sum over ranks: each rank's filter gradient covers only its strip
  size_t first = mgpu_->distributed() ? mgpu_->my_rank() : 0;
  mgpu_->allreduce_sum(sum_grad_[first].dptr(), param_dim_);
  const float mu = (float)cfg_.momentum->at(iter_count_);
  const float alpha = (float)cfg_.step_size->at(iter_count_);
  const float next_alpha = (float)cfg_.step_size->at(iter_count_ + 1);
  TxnId next;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    GPUConn conn = mgpu_->device_context(r)->conn();
    AD_CHECK(ad_sgd_step(param_dim_, param_[r].dptr(), sum_grad_[r].dptr(), momentum_[r].dptr(), (float)cfg_.l2_reg, mu, alpha,
                         next_alpha, cfg_.nesterov ? 1 : 0, nullptr, conn.stream()));
    any rd = param_[r];
    sink_->load_val(next, params_[r], 0, &rd);
  }
  ++iter_count_;
}

template <>
void ParallelSGDOptimizer<float>::store_params(size_t rank, float* host) {
  GPUConn conn = mgpu_->device_context(rank)->conn();
  param_[rank].store_sync(host, param_dim_, 0, conn);
}
template <>
void ParallelSGDOptimizer<float>::load_params(const float* host) {
  TxnId txn;
  for (size_t r = 0; r < mgpu_->num_ranks(); ++r) {
    if (!mgpu_->is_local(r)) continue;
    GPUConn conn = mgpu_->device_context(r)->conn();
    param_[r].load_sync(host, param_dim_, 0, conn);
    any rd = param_[r];
    sink_->load_val(txn, params_[r], 0, &rd);
    conn.sync();
  }
}
template <>
void ParallelSGDOptimizer<float>::store_sum_grads(size_t rank, float* host) {
  GPUConn conn = mgpu_->device_context(rank)->conn();
  sum_grad_[rank].store_sync(host, param_dim_, 0, conn);
}

}  // namespace arraydiff
