#include <cstdio>
#include <cstring>

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
    AD_CHECK(ad_sgd_step_guarded(param_dim_, param_[r].dptr(), sum_grad_[r].dptr(), momentum_[r].dptr(), (float)cfg_.l2_reg, mu, alpha,
                                 next_alpha, cfg_.nesterov ? 1 : 0, nullptr, mgpu_->device_context(r)->status_word(), conn.stream()));
    any rd = param_[r];
    sink_->load_val(next, params_[r], 0, &rd);
  }
  ++iter_count_;
}

// ------------------------------------------------------------------ the reference's calling convention
// reset(ctx) / step(compute_batch_fn, ctx): include/arraydiff/optimize.hh:314-564 of the reference.
template <>
void ParallelSGDOptimizer<float>::reset(shared_ptr<Context> parallel_ctx) {
  ctx_ = parallel_ctx;
  mgpu_ = dynamic_cast<MultiGPUContext*>(parallel_ctx.get());
  assert(mgpu_);
  const size_t R = mgpu_->num_ranks();
  if (batch_stats_.empty()) batch_stats_.resize(R);
  if (fixed_stats_.empty()) fixed_stats_.resize(R);
  TxnId init_txn;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    sink_->persist(init_txn, params_[r]);
    sink_->persist(init_txn, fixed_stats_[r]);
  }
  param_dim_ = 0; stat_dim_ = 0;
  bool have = false;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    const size_t d = sink_->store_val(init_txn, params_[r], 0, nullptr);
    const size_t sd = sink_->store_val(init_txn, fixed_stats_[r], 0, nullptr);
    assert(!have || (param_dim_ == d && stat_dim_ == sd));   // per-rank sub-graphs are built alike (reference :323-333)
    param_dim_ = d; stat_dim_ = sd; have = true;
    assert(sink_->store_grad(init_txn, grads_[r], 0, nullptr) == d);
    assert(sink_->store_val(init_txn, batch_stats_[r], 0, nullptr) == sd);
  }
  param_.resize(R); sum_grad_.resize(R); momentum_.resize(R);
  batch_grad_.resize(R); batch_stat_.resize(R); avg_stat_.resize(R); running_stat_.resize(R);
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    GPUContext* g = mgpu_->device_context(r).get();
    param_[r] = GPUMemory<float>(param_dim_, g);
    sum_grad_[r] = GPUMemory<float>(param_dim_, g);
    momentum_[r] = GPUMemory<float>(param_dim_, g);
    batch_grad_[r] = GPUMemory<float>(param_dim_, g);
    const size_t sd = stat_dim_ ? stat_dim_ : 1;
    batch_stat_[r] = GPUMemory<float>(sd, g);
    avg_stat_[r] = GPUMemory<float>(sd, g);
    running_stat_[r] = GPUMemory<float>(sd, g);
  }
  // rank 0's initial point and running statistics become everybody's (reference :358-386); ranks in other
  // processes drew from an equally seeded generator and hold the same values already
  const size_t first = mgpu_->distributed() ? mgpu_->my_rank() : 0;
  {
    any w = param_[first];
    sink_->store_val(init_txn, params_[first], 0, &w);
    any ws = running_stat_[first];
    if (stat_dim_) sink_->store_val(init_txn, fixed_stats_[first], 0, &ws);
  }
  mgpu_->device_context(first)->sync();
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r) || r == first) continue;
    GPUConn conn = mgpu_->device_context(r)->conn();
    CUDA_CHECK(cudaMemcpyAsync(param_[r].dptr(), param_[first].dptr(), param_dim_ * 4, cudaMemcpyDeviceToDevice, conn.stream()));
    if (stat_dim_)
      CUDA_CHECK(cudaMemcpyAsync(running_stat_[r].dptr(), running_stat_[first].dptr(), stat_dim_ * 4, cudaMemcpyDeviceToDevice, conn.stream()));
  }
  TxnId load_txn;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    any rd = param_[r];
    sink_->load_val(load_txn, params_[r], 0, &rd);
    any rs = running_stat_[r];
    if (stat_dim_) sink_->load_val(load_txn, fixed_stats_[r], 0, &rs);
  }
  iter_count_ = 0;
  mgpu_->sync();
}

template <>
void ParallelSGDOptimizer<float>::step(function<void(TxnId, size_t, shared_ptr<Op>)>& compute_batch_fn, shared_ptr<Context> parallel_ctx) {
  assert(mgpu_ && dynamic_cast<MultiGPUContext*>(parallel_ctx.get()) == mgpu_ && "reset(parallel_ctx) first");
  const size_t R = mgpu_->num_ranks();
  const size_t num_batches = (cfg_.minibatch_size + cfg_.compute_batch_size - 1) / cfg_.compute_batch_size;
  for (size_t b = 0; b < num_batches; ++b) {
    TxnId batch_txn;
    const size_t left = cfg_.minibatch_size - b * cfg_.compute_batch_size;
    compute_batch_fn(batch_txn, left < cfg_.compute_batch_size ? left : cfg_.compute_batch_size, sink_);
    for (size_t r = 0; r < R; ++r) {
      if (!mgpu_->is_local(r)) continue;
      GPUConn conn = mgpu_->device_context(r)->conn();
      // the first micro-batch writes the sums, the others add (reference :425-437)
      any gw = b == 0 ? sum_grad_[r] : batch_grad_[r];
      sink_->store_grad(batch_txn, grads_[r], 0, &gw);
      if (b) AD_CHECK(ad_array_add(param_dim_, batch_grad_[r].dptr(), sum_grad_[r].dptr(), conn.stream()));
      if (stat_dim_) {
        any sw = b == 0 ? avg_stat_[r] : batch_stat_[r];
        sink_->store_val(batch_txn, batch_stats_[r], 0, &sw);
        if (b) AD_CHECK(ad_array_add_online(stat_dim_, 1.0f / (float)(b + 1), batch_stat_[r].dptr(), avg_stat_[r].dptr(), conn.stream()));
      }
    }
  }
  // sum over ranks: each rank's filter gradient covers only its strip
  const size_t first = mgpu_->distributed() ? mgpu_->my_rank() : 0;
  mgpu_->allreduce_sum(sum_grad_[first].dptr(), param_dim_);
  const float mu = (float)cfg_.momentum->at(iter_count_);
  const float alpha = (float)cfg_.step_size->at(iter_count_);
  const float next_alpha = (float)cfg_.step_size->at(iter_count_ + 1);
  TxnId update_txn;
  for (size_t r = 0; r < R; ++r) {
    if (!mgpu_->is_local(r)) continue;
    GPUConn conn = mgpu_->device_context(r)->conn();
    AD_CHECK(ad_sgd_step_guarded(param_dim_, param_[r].dptr(), sum_grad_[r].dptr(), momentum_[r].dptr(), (float)cfg_.l2_reg, mu, alpha,
                                 next_alpha, cfg_.nesterov ? 1 : 0, nullptr, mgpu_->device_context(r)->status_word(), conn.stream()));
    any rd = param_[r];
    sink_->load_val(update_txn, params_[r], 0, &rd);
    if (stat_dim_) {
      // running += rate * (average batch statistic - running)   (reference :501-508)
      AD_CHECK(ad_array_add_online(stat_dim_, (float)cfg_.batch_norm_rate, avg_stat_[r].dptr(), running_stat_[r].dptr(), conn.stream()));
      any rs = running_stat_[r];
      sink_->load_val(update_txn, fixed_stats_[r], 0, &rs);
    }
  }
  ++iter_count_;
  mgpu_->end_phase();
}

// ------------------------------------------------------------------ checkpoint file
namespace {
struct File {
  FILE* f;
  explicit File(const string& path, const char* mode) : f(std::fopen(path.c_str(), mode)) {}
  ~File() { if (f) std::fclose(f); }
  template <typename V> bool put(const V& v) { return std::fwrite(&v, sizeof(V), 1, f) == 1; }
  template <typename V> bool get(V& v) { return std::fread(&v, sizeof(V), 1, f) == 1; }
};
const char kMagic[8] = {'A', 'D', 'B', '2', 'C', 'K', 'P', 'T'};
}  // namespace

template <>
bool ParallelSGDOptimizer<float>::save_checkpoint(const string& path) {
  assert(mgpu_ && "reset first");
  const size_t first = mgpu_->distributed() ? mgpu_->my_rank() : 0;
  ParamManifest man;
  {
    any w = &man;
    TxnId t;
    sink_->store_val(t, params_[first], 0, &w);
  }
  vector<float> theta(param_dim_), mom(param_dim_), stat(stat_dim_);
  {
    GPUConn conn = mgpu_->device_context(first)->conn();
    param_[first].store_sync(theta.data(), param_dim_, 0, conn);
    momentum_[first].store_sync(mom.data(), param_dim_, 0, conn);
    if (stat_dim_) running_stat_[first].store_sync(stat.data(), stat_dim_, 0, conn);
  }
  File out(path, "wb");
  if (!out.f) return false;
  bool ok = std::fwrite(kMagic, 1, 8, out.f) == 8 && out.put((uint32_t)1) && out.put((uint64_t)param_dim_) &&
            out.put((uint64_t)stat_dim_) && out.put((uint64_t)iter_count_) && out.put((uint32_t)man.size());
  for (auto& e : man) {
    ok = ok && out.put((uint32_t)e.name.size()) && std::fwrite(e.name.data(), 1, e.name.size(), out.f) == e.name.size() &&
         out.put((uint64_t)e.offset) && out.put((uint64_t)e.size);
  }
  ok = ok && std::fwrite(theta.data(), 4, param_dim_, out.f) == param_dim_ && std::fwrite(mom.data(), 4, param_dim_, out.f) == param_dim_ &&
       std::fwrite(stat.data(), 4, stat_dim_, out.f) == stat_dim_;
  return ok;
}

template <>
bool ParallelSGDOptimizer<float>::load_checkpoint(const string& path) {
  assert(mgpu_ && "reset first");
  File in(path, "rb");
  if (!in.f) return false;
  char magic[8];
  uint32_t version = 0, entries = 0;
  uint64_t pd = 0, sd = 0, it = 0;
  if (std::fread(magic, 1, 8, in.f) != 8 || std::memcmp(magic, kMagic, 8) || !in.get(version) || version != 1 || !in.get(pd) ||
      !in.get(sd) || !in.get(it) || !in.get(entries))
    return false;
  if (pd != param_dim_ || sd != stat_dim_) return false;
  const size_t first = mgpu_->distributed() ? mgpu_->my_rank() : 0;
  ParamManifest man;
  {
    any w = &man;
    TxnId t;
    sink_->store_val(t, params_[first], 0, &w);
  }
  if (entries != man.size()) return false;
  for (auto& e : man) {
    uint32_t len = 0;
    uint64_t off = 0, size = 0;
    if (!in.get(len) || len > 4096) return false;
    string name(len, ' ');
    if (std::fread(&name[0], 1, len, in.f) != len || !in.get(off) || !in.get(size)) return false;
    if (name != e.name || off != e.offset || size != e.size) return false;   // another net, or another build order
  }
  vector<float> theta(param_dim_), mom(param_dim_), stat(stat_dim_);
  if (std::fread(theta.data(), 4, param_dim_, in.f) != param_dim_ || std::fread(mom.data(), 4, param_dim_, in.f) != param_dim_ ||
      std::fread(stat.data(), 4, stat_dim_, in.f) != stat_dim_)
    return false;
  TxnId txn;
  for (size_t r = 0; r < mgpu_->num_ranks(); ++r) {
    if (!mgpu_->is_local(r)) continue;
    GPUConn conn = mgpu_->device_context(r)->conn();
    param_[r].load_sync(theta.data(), param_dim_, 0, conn);
    momentum_[r].load_sync(mom.data(), param_dim_, 0, conn);
    any rd = param_[r];
    sink_->load_val(txn, params_[r], 0, &rd);
    if (stat_dim_) {
      running_stat_[r].load_sync(stat.data(), stat_dim_, 0, conn);
      any rs = running_stat_[r];
      sink_->load_val(txn, fixed_stats_[r], 0, &rs);
    }
    conn.sync();
  }
  iter_count_ = (size_t)it;
  return true;
}

template <>
void ParallelSGDOptimizer<float>::broadcast_from_worker0() {
  assert(mgpu_ && mgpu_->distributed() && "reset first, on a context made with MakeDistributed");
  const size_t me = mgpu_->my_rank();
  GPUConn conn = mgpu_->device_context(me)->conn();
  const bool root = mgpu_->exchange_rank() == 0;
  if (!root) {
    AD_CHECK(ad_fill_zero(param_[me].dptr(), param_dim_ * 4, conn.stream()));
    if (stat_dim_) AD_CHECK(ad_fill_zero(running_stat_[me].dptr(), stat_dim_ * 4, conn.stream()));
  }
  mgpu_->allreduce_sum(param_[me].dptr(), param_dim_);       // x + 0 + ... + 0: worker 0's bits
  if (stat_dim_) mgpu_->allreduce_sum(running_stat_[me].dptr(), stat_dim_);
  TxnId txn;
  any rd = param_[me];
  sink_->load_val(txn, params_[me], 0, &rd);
  if (stat_dim_) {
    any rs = running_stat_[me];
    sink_->load_val(txn, fixed_stats_[me], 0, &rs);
  }
  mgpu_->end_phase();
  conn.sync();
}

template <>
void ParallelSGDOptimizer<float>::store_fixed_stats(size_t rank, float* host) {
  GPUConn conn = mgpu_->device_context(rank)->conn();
  if (stat_dim_) running_stat_[rank].store_sync(host, stat_dim_, 0, conn);
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
