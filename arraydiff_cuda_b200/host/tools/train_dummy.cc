// Training driver on synthetic data: the loop of the reference's tools/train_imagenet.cc:137-274 with DummyData
// (include/arraydiff/io/dummy.hh) in place of the ImageNet pipeline.  It builds the spatially parallel classifier
// through the op-graph API exactly the way the reference's tool does -- MultiGPUContext::Make, ResNet<float>::
// MakeParallelResNet18, op->init, ParallelSGDOptimizer(cfg, sum_loss, dev_params, dev_grads, dev_batch_stats,
// dev_fixed_stats), reset(ctx), step(batch_fn, ctx) with persist / load_val / gradient / store_val inside batch_fn --
// and prints the minibatch loss and accuracy of every iteration and a checksum of the final parameters.
//
//   ARRAYDIFF_B200_DEVICES=0,0 ARRAYDIFF_B200_MODE=bf16 train_dummy [iterations] [image] [batch] [minibatch] [resnet50]
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>

#include "arraydiff/context.hh"
#include "arraydiff/io/dummy.hh"
#include "arraydiff/optimize.hh"
#include "arraydiff/zoo.hh"

using namespace arraydiff;
using arraydiff::io::DummyData;

int main(int argc, char** argv) {
  const size_t train_iters = argc > 1 ? std::strtoul(argv[1], nullptr, 10) : 10;
  const size_t image = argc > 2 ? std::strtoul(argv[2], nullptr, 10) : 64;
  const size_t batch_size = argc > 3 ? std::strtoul(argv[3], nullptr, 10) : 8;
  const size_t minibatch_size = argc > 4 ? std::strtoul(argv[4], nullptr, 10) : 2 * batch_size;
  const bool deep = argc > 5 && !std::strcmp(argv[5], "resnet50");
  const size_t num_classes = 1000;

  DummyData<float> train_data(image, image, 3, 10, 1 << 20);
  size_t next_item = 0;

  auto parallel_ctx = MultiGPUContext::Make();
  ConvNetConfig net_cfg = {.input_w = image, .input_h = image, .batch_size = batch_size, .minibatch_size = minibatch_size};
  const size_t image_size = 3 * net_cfg.input_w * net_cfg.input_h;
  auto net = deep ? ResNet<float>::MakeParallelResNet50(net_cfg, parallel_ctx) : ResNet<float>::MakeParallelResNet18(net_cfg, parallel_ctx);
  parallel_ctx->sync();

  std::mt19937_64 init_rng(20240607);
  auto init_txn = TxnId();
  net.op->init(init_txn, &init_rng);

  const SGDConfig sgd_cfg = {
    .minibatch_size = minibatch_size,
    .compute_batch_size = batch_size,
    .step_size = make_shared<PiecewiseStepSchedule<double>>(0.05, train_iters * 2 / 3, 0.005),
    .momentum = make_shared<ConstantSchedule<double>>(0.9),
    .nesterov = true,
    .l2_reg = 1.0e-4,
    .batch_norm_rate = 0.003,
  };
  ParallelSGDOptimizer<float> sgd(sgd_cfg, net.sum_loss, net.dev_params, net.dev_grads, net.dev_batch_stats, net.dev_fixed_stats);
  sgd.reset(parallel_ctx);

  vector<float> batch_input(image_size * batch_size), batch_logit(num_classes * batch_size), batch_loss(batch_size);
  vector<uint32_t> batch_label(batch_size);

  for (size_t t = 0; t < train_iters; ++t) {
    auto start = std::chrono::steady_clock::now();
    float correct = 0.0f, loss_sum = 0.0f;
    auto batch_fn = static_cast<function<void(TxnId, size_t, shared_ptr<Op>)>>(
        [&](TxnId batch_txn, size_t batch, shared_ptr<Op> loss) {
          *net.batch_norm_use_fixed = false;
          const size_t num_ranks = parallel_ctx->num_ranks();
          for (size_t rank = 0; rank < num_ranks; ++rank) {
            loss->persist(batch_txn, net.dev_params.at(rank));
            loss->persist(batch_txn, net.dev_fixed_stats.at(rank));
          }
          for (size_t idx = 0; idx < batch; ++idx) {
            auto item = train_data.at(next_item++ % train_data.size());
            std::memcpy(batch_input.data() + image_size * idx, item.first.buffer, sizeof(float) * image_size);
            item.first.dealloc();
            batch_label[idx] = item.second;
          }
          any input_reader(Slice<float>(batch_input.data(), image_size * batch));
          size_t input_offset = loss->load_val(batch_txn, net.inputs, 0, &input_reader);
          assert(image_size * batch == input_offset);
          any label_reader(Slice<uint32_t>(batch_label.data(), batch));
          size_t label_offset = loss->load_val(batch_txn, net.labels, 0, &label_reader);
          assert(batch == label_offset);

          loss->gradient(batch_txn);
          parallel_ctx->sync();

          any logit_writer(Slice<float>(batch_logit.data(), num_classes * batch));
          size_t logit_offset = loss->store_val(batch_txn, net.logits, 0, &logit_writer);
          assert(num_classes * batch == logit_offset);
          for (size_t idx = 0; idx < batch; ++idx) {
            size_t best = 0;
            for (size_t k = 1; k < num_classes; ++k)
              if (batch_logit[k + num_classes * idx] > batch_logit[best + num_classes * idx]) best = k;
            if (best == batch_label[idx]) correct += 1.0f;
          }
          any loss_writer(Slice<float>(batch_loss.data(), batch));
          size_t loss_offset = loss->store_val(batch_txn, net.losses, 0, &loss_writer);
          assert(batch == loss_offset);
          for (size_t idx = 0; idx < batch; ++idx) loss_sum += batch_loss[idx];
          (void)input_offset; (void)label_offset; (void)logit_offset; (void)loss_offset;
        });
    sgd.step(batch_fn, parallel_ctx);
    parallel_ctx->sync();
    double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - start).count();
    std::printf("iter %zu loss %.6f accuracy %.4f lr %g elapsed_ms %.2f\n", t, loss_sum / (float)minibatch_size,
                correct / (float)minibatch_size, sgd_cfg.step_size->at(t), ms);
  }

  // validation pass on the running statistics (the switch the reference's tools flip for their validation runs)
  {
    *net.batch_norm_use_fixed = true;
    TxnId val_txn;
    for (size_t rank = 0; rank < parallel_ctx->num_ranks(); ++rank) {
      net.sum_loss->persist(val_txn, net.dev_params.at(rank));
      net.sum_loss->persist(val_txn, net.dev_fixed_stats.at(rank));
    }
    any input_reader(Slice<float>(batch_input.data(), image_size * batch_size));
    net.sum_loss->load_val(val_txn, net.inputs, 0, &input_reader);
    any label_reader(Slice<uint32_t>(batch_label.data(), batch_size));
    net.sum_loss->load_val(val_txn, net.labels, 0, &label_reader);
    net.sum_loss->eval(val_txn);
    parallel_ctx->sync();
    any loss_writer(Slice<float>(batch_loss.data(), batch_size));
    net.sum_loss->store_val(val_txn, net.losses, 0, &loss_writer);
    double s = 0.0;
    for (size_t idx = 0; idx < batch_size; ++idx) s += batch_loss[idx];
    std::printf("validation_loss_fixed_stats %.6f\n", s / (double)batch_size);
    *net.batch_norm_use_fixed = false;
  }

  vector<float> params(sgd.param_dim()), stats(sgd.stat_dim() ? sgd.stat_dim() : 1);
  double checksum = 0.0, abs_sum = 0.0;
  for (size_t rank = 0; rank < parallel_ctx->num_ranks(); ++rank) {
    sgd.store_params(rank, params.data());
    double c = 0.0;
    for (float v : params) { c += (double)v; if (rank == 0) abs_sum += std::fabs((double)v); }
    if (rank == 0) checksum = c;
    else if (c != checksum) { std::printf("rank %zu parameters differ from rank 0\n", rank); return 2; }
  }
  sgd.store_fixed_stats(0, stats.data());
  double stat_sum = 0.0;
  for (size_t i = 0; i < sgd.stat_dim(); ++i) stat_sum += (double)stats[i];
  std::printf("params %zu checksum %.9e abs %.9e stat_dim %zu stat_sum %.9e status %d\n", sgd.param_dim(), checksum, abs_sum,
              sgd.stat_dim(), stat_sum, parallel_ctx->device_context(0)->read_status());
  return 0;
}
