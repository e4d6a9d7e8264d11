// Builders: every function creates the same operators in the same order on every rank.
#include <cmath>

#include "arraydiff/zoo.hh"

namespace arraydiff {

static size_t ranks_of(const shared_ptr<Context>& ctx) {
  auto m = dynamic_cast<MultiGPUContext*>(ctx.get());
  return m ? m->num_ranks() : 1;
}
static GPUContext* gpu_at(const shared_ptr<Context>& ctx, size_t rank) {
  if (auto m = dynamic_cast<MultiGPUContext*>(ctx.get())) return m->device_context(rank).get();
  return dynamic_cast<GPUContext*>(ctx.get());
}
static bool local_rank(const shared_ptr<Context>& ctx, size_t rank) {
  auto m = dynamic_cast<MultiGPUContext*>(ctx.get());
  return m ? m->is_local(rank) : true;
}

template <typename A>
typename IOOp<A>::InitFn kaiming_init_gen(size_t fan_in, size_t) {
  return [fan_in](A* a, std::mt19937_64* rng, shared_ptr<Context>) {
    std::normal_distribution<float> dist(0.0f, std::sqrt(2.0f / (float)fan_in));
    vector<float> h(a->flat_size());
    for (auto& v : h) v = dist(*rng);
    // the context streams do not synchronise with the default stream: drain what is queued on this
    // array (its allocation-time zero fill) before the copy, and the copy before anything reads it
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(a->dptr(), h.data(), h.size() * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaDeviceSynchronize());
  };
}
template <typename A>
typename IOOp<A>::InitFn xavier_init_gen(size_t fan_in, size_t fan_out) {
  return [fan_in, fan_out](A* a, std::mt19937_64* rng, shared_ptr<Context>) {
    const float half = std::sqrt(6.0f / (float)(fan_in + fan_out));
    std::uniform_real_distribution<float> dist(-half, half);
    vector<float> h(a->flat_size());
    for (auto& v : h) v = dist(*rng);
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(a->dptr(), h.data(), h.size() * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaDeviceSynchronize());
  };
}
template <typename A>
typename IOOp<A>::InitFn zeros_init_gen() {
  return [](A* a, std::mt19937_64*, shared_ptr<Context>) {
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemset(a->dptr(), 0, a->flat_size() * 4));
    CUDA_CHECK(cudaDeviceSynchronize());
  };
}
template IOOp<GPUArray4D<float>>::InitFn kaiming_init_gen<GPUArray4D<float>>(size_t, size_t);
template IOOp<GPUArray1D<float>>::InitFn zeros_init_gen<GPUArray1D<float>>();
template IOOp<GPUArray4D<float>>::InitFn xavier_init_gen<GPUArray4D<float>>(size_t, size_t);

template <>
ParamOp<Act> conv2d(Conv2DShape shape, ActVar input, KernelInitFn kernel_init, bool enable_bias, shared_ptr<Context> ctx) {
  const size_t r = input->rank();
  const size_t cin = input->shape().shape[2];
  // Shape4D(kw, kh, c_in, c_out): KCRS in memory (reference src/zoo.cc:102)
  auto kernel = IOOp<GPUArray4D<float>>::Make(Shape4D(shape.kernel[0], shape.kernel[1], cin, shape.filters), 1, kernel_init, r, ctx);
  shared_ptr<IOOp<GPUArray1D<float>>> bias;
  if (enable_bias) bias = IOOp<GPUArray1D<float>>::Make(Shape1D(shape.filters), 1, zeros_init_gen<GPUArray1D<float>>(), r, ctx);
  kernel->set_name(NameScope::current() + ".kernel");
  if (bias) bias->set_name(NameScope::current() + ".bias");
  ParamOp<Act> p;
  p.op = CudnnConv2DOpF::Make(shape, input, kernel, bias, ctx);
  p.params.insert(kernel->data().val.var());
  p.grads.insert(kernel->data().grad.var());
  if (bias) { p.params.insert(bias->data().val.var()); p.grads.insert(bias->data().grad.var()); }
  return p;
}

template <>
ParallelParamOp<Act> parallel_conv2d(Conv2DShape shape, vector<ActVar> inputs, KernelInitFn kernel_init, bool enable_bias,
                                     shared_ptr<Context> ctx) {
  ParallelParamOp<Act> out;
  for (auto& x : inputs) {   // one op per rank, each with its own parameter variable (reference src/zoo.cc:140-153)
    auto p = conv2d<Act>(shape, x, kernel_init, enable_bias, ctx);
    out.ops.push_back(p.op);
    out.params.push_back(p.params);
    out.grads.push_back(p.grads);
  }
  return out;
}

template <>
ParamOp<Act> linear(size_t filters, ActVar input, KernelInitFn kernel_init, shared_ptr<Context> ctx) {
  const size_t r = input->rank();
  const size_t in = input->shape().shape[2];
  // Shape4D(1, 1, in, out): [out][in] in memory, the reference's Shape2D(in, out)
  auto kernel = IOOp<GPUArray4D<float>>::Make(Shape4D(1, 1, in, filters), 1, kernel_init, r, ctx);
  auto bias = IOOp<GPUArray1D<float>>::Make(Shape1D(filters), 1, zeros_init_gen<GPUArray1D<float>>(), r, ctx);
  kernel->set_name(NameScope::current() + ".kernel");
  bias->set_name(NameScope::current() + ".bias");
  ParamOp<Act> p;
  p.op = CublasLinearOpF::Make(filters, input, kernel, bias, ctx);
  p.params.insert(kernel->data().val.var()); p.params.insert(bias->data().val.var());
  p.grads.insert(kernel->data().grad.var()); p.grads.insert(bias->data().grad.var());
  return p;
}
template <>
ParallelParamOp<Act> parallel_linear(size_t filters, vector<ActVar> inputs, KernelInitFn kernel_init, shared_ptr<Context> ctx) {
  ParallelParamOp<Act> out;
  for (auto& x : inputs) {
    auto p = linear<Act>(filters, x, kernel_init, ctx);
    out.ops.push_back(p.op);
    out.params.push_back(p.params);
    out.grads.push_back(p.grads);
  }
  return out;
}

template <>
vector<ActVar> parallel_relu(vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (auto& x : inputs) out.push_back(CudnnActivationOpF::Make(kReluAct, x, ctx));
  return out;
}
template <>
vector<ActVar> parallel_sum(vector<vector<ActVar>> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (size_t r = 0; r < inputs.at(0).size(); ++r) {
    vector<ActVar> xs;
    for (auto& branch : inputs) xs.push_back(branch.at(r));
    out.push_back(SumJoinOpF::Make(xs, ctx));
  }
  return out;
}
template <>
ParallelBatchNormParamOp<Act> parallel_batch_norm(size_t channels, shared_ptr<bool> switch_var, vector<ActVar> inputs, bool fuse_relu,
                                                  shared_ptr<Context> ctx) {
  ParallelBatchNormParamOp<Act> out;
  for (auto& x : inputs) {
    auto parts = CudnnBatchNorm2DOpF::Make(channels, switch_var, x, ctx);
    if (fuse_relu) parts.op->fuse_relu();
    out.ops.push_back(parts.op);
    VarIdSet p, g, bs, fs;
    p.insert(parts.scale->data().val.var()); p.insert(parts.shift->data().val.var());
    g.insert(parts.scale->data().grad.var()); g.insert(parts.shift->data().grad.var());
    bs.insert(parts.batch_mean->data().val.var()); bs.insert(parts.batch_variance->data().val.var());
    fs.insert(parts.fixed_mean->data().val.var()); fs.insert(parts.fixed_variance->data().val.var());
    out.params.push_back(p); out.grads.push_back(g); out.batch_stats.push_back(bs); out.fixed_stats.push_back(fs);
  }
  return out;
}

// Collects the per-rank variable sets while a block is assembled.
struct BlockVars {
  explicit BlockVars(size_t R) : params(R), grads(R), batch_stats(R), fixed_stats(R) {}
  void add(const ParallelParamOp<Act>& p) {
    for (size_t r = 0; r < params.size(); ++r) { params[r].insert_all(p.params[r]); grads[r].insert_all(p.grads[r]); }
  }
  void add(const ParallelBatchNormParamOp<Act>& p) {
    for (size_t r = 0; r < params.size(); ++r) {
      params[r].insert_all(p.params[r]); grads[r].insert_all(p.grads[r]);
      batch_stats[r].insert_all(p.batch_stats[r]); fixed_stats[r].insert_all(p.fixed_stats[r]);
    }
  }
  ParallelBatchNormParamOp<Act> finish(vector<ActVar> ops) { return {ops, params, grads, batch_stats, fixed_stats}; }
  vector<VarIdSet> params, grads, batch_stats, fixed_stats;
};

// BN -> ReLU, fused into one kernel
static vector<ActVar> bn_relu(const char* name, size_t channels, shared_ptr<bool> sw, vector<ActVar> in, BlockVars& vars, shared_ptr<Context> ctx) {
  NameScope scope(name);
  auto bn = parallel_batch_norm<Act>(channels, sw, in, true, ctx);
  vars.add(bn);
  return bn.ops;
}
// halo pad -> halo exchange -> conv on the halo-padded strip
static vector<ActVar> halo_conv(const char* name, Conv2DShape shape, vector<ActVar> in, BlockVars& vars, shared_ptr<Context> ctx) {
  NameScope scope(name);
  assert(shape.pad[0] == shape.pad[1]);
  shape.halo_padded_input = true;
  auto pad = HaloPad2DOpF::MakeParallel(shape.pad[0], in, ctx);
  auto exch = HaloExch2DOpF::MakeParallel(shape.pad[0], pad, ctx);
  const size_t cin = in.at(0)->shape().shape[2];
  auto conv = parallel_conv2d<Act>(shape, exch, kaiming_init_gen<GPUArray4D<float>>(cin * shape.kernel[0] * shape.kernel[1], shape.filters), false, ctx);
  vars.add(conv);
  return conv.ops;
}
static vector<ActVar> conv1x1(const char* name, size_t filters, size_t stride, vector<ActVar> in, BlockVars& vars, shared_ptr<Context> ctx) {
  NameScope scope(name);
  Conv2DShape s;
  s.filters = filters; s.kernel = {1, 1}; s.stride = {stride, stride}; s.pad = {0, 0};
  auto conv = parallel_conv2d<Act>(s, in, kaiming_init_gen<GPUArray4D<float>>(in.at(0)->shape().shape[2], filters), false, ctx);
  vars.add(conv);
  return conv.ops;
}

// BN-ReLU-[pad-exch-conv3x3] x2, identity shortcut   (reference src/zoo.cc:577-652)
template <>
ParallelBatchNormParamOp<Act> spatial_parallel_residual_v2_conv2d(Conv2DShape shape, shared_ptr<bool> sw, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  BlockVars vars(inputs.size());
  shape.stride = {1, 1};
  auto a0 = bn_relu("bn0", inputs.at(0)->shape().shape[2], sw, inputs, vars, ctx);
  auto c1 = halo_conv("conv1", shape, a0, vars, ctx);
  auto a1 = bn_relu("bn1", shape.filters, sw, c1, vars, ctx);
  auto c2 = halo_conv("conv2", shape, a1, vars, ctx);
  return vars.finish(parallel_sum<Act>({inputs, c2}, ctx));
}
// same with a strided 1x1 projection shortcut taken after the first BN-ReLU   (reference src/zoo.cc:654-738)
template <>
ParallelBatchNormParamOp<Act> spatial_parallel_proj_residual_v2_conv2d(Conv2DShape shape, size_t stride, shared_ptr<bool> sw, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  BlockVars vars(inputs.size());
  auto a0 = bn_relu("bn0", inputs.at(0)->shape().shape[2], sw, inputs, vars, ctx);
  auto proj = conv1x1("proj", shape.filters, stride, a0, vars, ctx);
  Conv2DShape s1 = shape;
  s1.stride = {stride, stride};
  auto c1 = halo_conv("conv1", s1, a0, vars, ctx);
  auto a1 = bn_relu("bn1", shape.filters, sw, c1, vars, ctx);
  Conv2DShape s2 = shape;
  s2.stride = {1, 1};
  auto c2 = halo_conv("conv2", s2, a1, vars, ctx);
  return vars.finish(parallel_sum<Act>({proj, c2}, ctx));
}
// BN-ReLU-1x1, BN-ReLU-[pad-exch-3x3], BN-ReLU-1x1 (x bottleneck), identity shortcut   (reference src/zoo.cc:740-837)
template <>
ParallelBatchNormParamOp<Act> spatial_parallel_bottleneck_residual_v2_conv2d(Conv2DShape shape, size_t bottleneck, shared_ptr<bool> sw, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  BlockVars vars(inputs.size());
  assert(inputs.at(0)->shape().shape[2] == bottleneck * shape.filters);   // channels are axis 2
  shape.stride = {1, 1};
  auto a0 = bn_relu("bn0", inputs.at(0)->shape().shape[2], sw, inputs, vars, ctx);
  auto c1 = conv1x1("conv1", shape.filters, 1, a0, vars, ctx);
  auto a1 = bn_relu("bn1", shape.filters, sw, c1, vars, ctx);
  auto c2 = halo_conv("conv2", shape, a1, vars, ctx);
  auto a2 = bn_relu("bn2", shape.filters, sw, c2, vars, ctx);
  auto c3 = conv1x1("conv3", bottleneck * shape.filters, 1, a2, vars, ctx);
  return vars.finish(parallel_sum<Act>({inputs, c3}, ctx));
}
// bottleneck with a strided 1x1 projection shortcut; the 3x3 carries the stride   (reference src/zoo.cc:839-946,
// which strides only the projection: the single-GPU twin at :541-542 strides the 3x3 as done here)
template <>
ParallelBatchNormParamOp<Act> spatial_parallel_proj_bottleneck_residual_v2_conv2d(Conv2DShape shape, size_t bottleneck, size_t stride, shared_ptr<bool> sw, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  BlockVars vars(inputs.size());
  auto a0 = bn_relu("bn0", inputs.at(0)->shape().shape[2], sw, inputs, vars, ctx);
  auto proj = conv1x1("proj", bottleneck * shape.filters, stride, a0, vars, ctx);
  auto c1 = conv1x1("conv1", shape.filters, 1, a0, vars, ctx);
  auto a1 = bn_relu("bn1", shape.filters, sw, c1, vars, ctx);
  Conv2DShape s2 = shape;
  s2.stride = {stride, stride};
  auto c2 = halo_conv("conv2", s2, a1, vars, ctx);
  auto a2 = bn_relu("bn2", shape.filters, sw, c2, vars, ctx);
  auto c3 = conv1x1("conv3", bottleneck * shape.filters, 1, a2, vars, ctx);
  return vars.finish(parallel_sum<Act>({proj, c3}, ctx));
}

// scatter_on_load: every rank's input variable is its strip, filled straight from the host image (HostRows);
// otherwise every rank holds the whole image and a SpatialScatter2DOp cuts out its rows inside the graph
// (the reference's BroadcastOp + SpatialScatter2DOp, src/zoo.cc:1522-1523).
static SpatialParallelNet begin_net(const ConvNetConfig& cfg, shared_ptr<Context> ctx, vector<ActVar>& strips, bool scatter_on_load = false) {
  SpatialParallelNet net;
  const size_t R = ranks_of(ctx);
  net.batch_norm_use_fixed = make_shared<bool>(false);
  net.dev_params.resize(R); net.dev_grads.resize(R); net.dev_batch_stats.resize(R); net.dev_fixed_stats.resize(R);
  net.output_grad_vars.resize(R);
  assert(cfg.input_h % R == 0);
  vector<ActVar> full;
  for (size_t r = 0; r < R; ++r) {
    if (!local_rank(ctx, r)) { net.inputs.push_back(nullptr); continue; }
    auto in = IOOp<Act>::Make(Shape3D(cfg.input_w, scatter_on_load ? cfg.input_h / R : cfg.input_h, cfg.input_c), cfg.batch_size, nullptr, r, ctx);
    net.inputs.push_back(in);
    net.input_vars.insert(in->data().val.var());
    full.push_back(in);
  }
  if (scatter_on_load) { strips = full; return net; }
  // every rank holds the image and cuts out its own rows (reference src/zoo.cc:1522-1523)
  for (auto& x : full) strips.push_back(make_shared<SpatialScatter2DOpF>(x->rank(), R, x, ctx));
  (void)gpu_at;
  return net;
}
static void absorb(SpatialParallelNet& net, const vector<ActVar>& ops, const vector<VarIdSet>& p, const vector<VarIdSet>& g,
                   const vector<VarIdSet>* bs = nullptr, const vector<VarIdSet>* fs = nullptr) {
  for (size_t i = 0; i < ops.size(); ++i) {
    const size_t r = ops[i]->rank();
    net.dev_params[r].insert_all(p[i]); net.dev_grads[r].insert_all(g[i]);
    if (bs) net.dev_batch_stats[r].insert_all((*bs)[i]);
    if (fs) net.dev_fixed_stats[r].insert_all((*fs)[i]);
  }
}
static void finish_net(SpatialParallelNet& net, const vector<ActVar>& outs) {
  net.outputs = outs;
  vector<shared_ptr<Op>> members(outs.begin(), outs.end());
  net.sink = make_shared<GroupSinkOp>(members);
  for (auto& o : outs) net.output_grad_vars[o->rank()].insert(o->data().grad.var());
}

template <>
SpatialParallelNet SpatialParallelResNet<float>::MakeConv3x3(const ConvNetConfig& cfg, size_t filters, shared_ptr<Context> ctx,
                                                             size_t first_pad) {
  vector<ActVar> strips;
  SpatialParallelNet net = begin_net(cfg, ctx, strips);
  Conv2DShape s;
  s.filters = filters; s.kernel = {3, 3}; s.pad = {1, 1}; s.halo_padded_input = true;
  auto pad = HaloPad2DOpF::MakeParallel(first_pad, strips, ctx);
  // a wider first frame is moved into the 1-pixel frame the layer reads (what a net does between a halo-3 and a halo-1
  // layer that share an input, reference HaloRepad2DOp, include/arraydiff/op.hh:2548)
  if (first_pad != 1) pad = HaloRepad2DOpF::MakeParallel(first_pad, 1, pad, ctx);
  auto exch = HaloExch2DOpF::MakeParallel(1, pad, ctx);
  NameScope scope("conv");
  auto conv = parallel_conv2d<Act>(s, exch, kaiming_init_gen<GPUArray4D<float>>(cfg.input_c * 9, filters), false, ctx);
  absorb(net, conv.ops, conv.params, conv.grads);
  // grads of the input are wanted too in this plumbing case: an IOOp keeps them
  finish_net(net, conv.ops);
  return net;
}

// The same layer written the reference's way (src/zoo.cc:1522-1523, :1841-1842, :1873): the image lives on rank 0 and is
// broadcast, every rank cuts out its strip inside the graph, the strips of the result are placed into zeroed full
// tensors and all-reduced (= all-gathered), and the replicas are reduced to rank 0.  The single output is therefore
// R times the convolution of the whole image.  One-process contexts only.
template <>
SpatialParallelNet SpatialParallelResNet<float>::MakeConv3x3Collectives(const ConvNetConfig& cfg, size_t filters, shared_ptr<Context> ctx) {
  SpatialParallelNet net;
  const size_t R = ranks_of(ctx);
  net.batch_norm_use_fixed = make_shared<bool>(false);
  net.dev_params.resize(R); net.dev_grads.resize(R); net.dev_batch_stats.resize(R); net.dev_fixed_stats.resize(R);
  net.output_grad_vars.resize(R);
  auto in = IOOp<Act>::Make(Shape3D(cfg.input_w, cfg.input_h, cfg.input_c), cfg.batch_size, nullptr, 0, ctx);
  net.inputs.assign(R, nullptr);
  net.inputs[0] = in;
  net.input_vars.insert(in->data().val.var());
  auto everywhere = BroadcastOp<Act>::MakeParallel(0, in, ctx);
  auto strips = SpatialScatter2DOp<Act>::MakeParallel(everywhere, ctx);
  Conv2DShape s;
  s.filters = filters; s.kernel = {3, 3}; s.pad = {1, 1}; s.halo_padded_input = true;
  auto pad = HaloPad2DOp<Act>::MakeParallel(1, strips, ctx);
  auto exch = HaloExch2DOp<Act>::MakeParallel(1, pad, ctx);
  ParallelParamOp<Act> conv;
  { NameScope scope("conv"); conv = parallel_conv2d<Act>(s, exch, kaiming_init_gen<GPUArray4D<float>>(cfg.input_c * 9, filters), false, ctx); }
  absorb(net, conv.ops, conv.params, conv.grads);
  auto placed = SpatialGather2DOp<Act>::MakeParallel(conv.ops, ctx);
  auto full = AllreduceOp<Act>::MakeParallel(placed, ctx);
  ActVar total = ReduceOp<Act>::MakeParallel(0, full, ctx);
  net.outputs = {total};
  net.sink = make_shared<GroupSinkOp>(vector<shared_ptr<Op>>{total});
  net.output_grad_vars[0].insert(total->data().grad.var());
  return net;
}

// ResNet stem on H-strips: halo 3, 7x7/2 -> `width` channels, BN + ReLU, then a 3x3/2 max pool on a halo-1 strip
static vector<ActVar> stem(SpatialParallelNet& net, const ConvNetConfig& cfg, size_t width, vector<ActVar> strips, shared_ptr<Context> ctx) {
  auto sw = net.batch_norm_use_fixed;
  Conv2DShape c1;
  c1.filters = width; c1.kernel = {7, 7}; c1.stride = {2, 2}; c1.pad = {3, 3}; c1.halo_padded_input = true;
  auto pad1 = HaloPad2DOpF::MakeParallel(3, strips, ctx);
  auto exch1 = HaloExch2DOpF::MakeParallel(3, pad1, ctx);
  ParallelParamOp<Act> conv1;
  { NameScope scope("stem.conv"); conv1 = parallel_conv2d<Act>(c1, exch1, kaiming_init_gen<GPUArray4D<float>>(cfg.input_c * 49, width), false, ctx); }
  absorb(net, conv1.ops, conv1.params, conv1.grads);
  ParallelBatchNormParamOp<Act> bn1;
  { NameScope scope("stem.bn"); bn1 = parallel_batch_norm<Act>(width, sw, conv1.ops, true, ctx); }
  absorb(net, bn1.ops, bn1.params, bn1.grads, &bn1.batch_stats, &bn1.fixed_stats);
  Pool2DShape pool;
  pool.window = {3, 3}; pool.stride = {2, 2}; pool.pad = {1, 1}; pool.halo_padded_input = true;
  auto pad2 = HaloPad2DOpF::MakeParallel(1, bn1.ops, ctx);
  auto exch2 = HaloExch2DOpF::MakeParallel(1, pad2, ctx);
  return CudnnPool2DOpF::MakeParallel(pool, exch2, ctx);
}

template <>
SpatialParallelNet SpatialParallelResNet<float>::MakeStemStage1(const ConvNetConfig& cfg, shared_ptr<Context> ctx) {
  vector<ActVar> strips;
  SpatialParallelNet net = begin_net(cfg, ctx, strips, true);
  auto sw = net.batch_norm_use_fixed;
  auto pooled = stem(net, cfg, 64, strips, ctx);
  // stage 1: bottlenecks 64-64-256
  Conv2DShape b;
  b.filters = 64; b.kernel = {3, 3}; b.pad = {1, 1};
  ParallelBatchNormParamOp<Act> blk;
  { NameScope scope("block1"); blk = spatial_parallel_proj_bottleneck_residual_v2_conv2d<Act>(b, 4, 1, sw, pooled, ctx); }
  absorb(net, blk.ops, blk.params, blk.grads, &blk.batch_stats, &blk.fixed_stats);
  for (int i = 0; i < 2; ++i) {
    NameScope scope(i == 0 ? "block2" : "block3");
    blk = spatial_parallel_bottleneck_residual_v2_conv2d<Act>(b, 4, sw, blk.ops, ctx);
    absorb(net, blk.ops, blk.params, blk.grads, &blk.batch_stats, &blk.fixed_stats);
  }
  finish_net(net, blk.ops);
  return net;
}

// Dilated ResNet-50 for per-pixel classification at output stride 8: stem, stages of pre-activation
// bottlenecks (stage 2 strided, stages 3 and 4 dilated by 2 and 4 with halos of 2 and 4 rows), BN + ReLU,
// 1x1 classifier with bias, x8 bilinear upsample of the halo-1 logits, per-pixel softmax NLL.
// Built from the same spatial_parallel_* blocks as the reference's nets (src/zoo.cc:740-946); the head is
// the one its CudnnSoftmaxNLLLossOp stops short of (src/op.cc:4225).
template <>
SpatialParallelNet SpatialParallelResNet<float>::MakeSegNet50(const ConvNetConfig& cfg, const SegNetConfig& seg, shared_ptr<Context> ctx) {
  vector<ActVar> strips;
  SpatialParallelNet net = begin_net(cfg, ctx, strips, true);
  auto sw = net.batch_norm_use_fixed;
  vector<ActVar> cur = stem(net, cfg, seg.base, strips, ctx);
  const size_t strides[4] = {1, 2, 1, 1}, dils[4] = {1, 1, 2, 4};
  for (int st = 0; st < 4; ++st) {
    Conv2DShape b;
    b.filters = seg.base << st; b.kernel = {3, 3}; b.dilate = {dils[st], dils[st]}; b.pad = {dils[st], dils[st]};
    for (size_t i = 0; i < seg.blocks[st]; ++i) {
      NameScope scope("stage" + std::to_string(st + 1) + ".block" + std::to_string(i + 1));
      ParallelBatchNormParamOp<Act> blk =
          i == 0 ? spatial_parallel_proj_bottleneck_residual_v2_conv2d<Act>(b, 4, strides[st], sw, cur, ctx)
                 : spatial_parallel_bottleneck_residual_v2_conv2d<Act>(b, 4, sw, cur, ctx);
      absorb(net, blk.ops, blk.params, blk.grads, &blk.batch_stats, &blk.fixed_stats);
      cur = blk.ops;
    }
  }
  ParallelBatchNormParamOp<Act> bnf;
  { NameScope scope("head.bn"); bnf = parallel_batch_norm<Act>((seg.base << 3) * 4, sw, cur, true, ctx); }
  absorb(net, bnf.ops, bnf.params, bnf.grads, &bnf.batch_stats, &bnf.fixed_stats);
  Conv2DShape hc;
  hc.filters = seg.classes; hc.kernel = {1, 1};
  ParallelParamOp<Act> head;
  { NameScope scope("head.conv"); head = parallel_conv2d<Act>(hc, bnf.ops, kaiming_init_gen<GPUArray4D<float>>((seg.base << 3) * 4, seg.classes), true, ctx); }
  absorb(net, head.ops, head.params, head.grads);
  auto padl = HaloPad2DOpF::MakeParallel(1, head.ops, ctx);
  auto exchl = HaloExch2DOpF::MakeParallel(1, padl, ctx);
  auto up = UpsampleBilinear2DOpF::MakeParallel(8, exchl, ctx);
  net.losses = CudnnSoftmaxNLLLoss2DOpF::MakeParallel(up, ctx);
  size_t pixels = 0;
  const size_t R = ranks_of(ctx);
  for (auto& l : net.losses) pixels = l->pixels() * R;   // equal strips
  for (auto& l : net.losses) l->set_loss_weight(1.0f / (float)pixels);   // gradient of the mean loss over the whole batch
  net.outputs = up;
  vector<shared_ptr<Op>> members(net.losses.begin(), net.losses.end());
  net.sink = make_shared<GroupSinkOp>(members);
  for (auto& o : up) net.output_grad_vars[o->rank()].insert(o->data().grad.var());
  return net;
}

template <>
SpatialParallelNet SpatialParallelResNet<float>::MakeParallelResNet18(const ConvNetConfig& cfg, size_t classes, shared_ptr<Context> ctx) {
  vector<ActVar> strips;
  SpatialParallelNet net = begin_net(cfg, ctx, strips, true);
  auto sw = net.batch_norm_use_fixed;
  const size_t R = ranks_of(ctx);
  // conv1: 7x7, stride 1, bias, Xavier (reference src/zoo.cc:1527-1556); no BN / ReLU before the pool
  Conv2DShape c1;
  c1.filters = 64; c1.kernel = {7, 7}; c1.pad = {3, 3}; c1.halo_padded_input = true;
  auto pad1 = HaloPad2DOpF::MakeParallel(3, strips, ctx);
  auto exch1 = HaloExch2DOpF::MakeParallel(3, pad1, ctx);
  ParallelParamOp<Act> conv1;
  { NameScope scope("conv1"); conv1 = parallel_conv2d<Act>(c1, exch1, xavier_init_gen<GPUArray4D<float>>(cfg.input_c * 49, 64), true, ctx); }
  absorb(net, conv1.ops, conv1.params, conv1.grads);
  Pool2DShape pool;
  pool.window = {3, 3}; pool.stride = {2, 2}; pool.pad = {1, 1}; pool.halo_padded_input = true;
  auto pad2 = HaloPad2DOpF::MakeParallel(1, conv1.ops, ctx);
  auto exch2 = HaloExch2DOpF::MakeParallel(1, pad2, ctx);
  vector<ActVar> cur = CudnnPool2DOpF::MakeParallel(pool, exch2, ctx);
  // res2_1, res2_2 (64) | res3_1 (128, /2), res3_2 | res4_1 (256, /2), res4_2 | res5_1 (512, /2) | res6_1 (512, /2)
  struct Blk { const char* name; size_t filters; bool proj; };
  const Blk blocks[] = {{"res2_1", 64, false}, {"res2_2", 64, false}, {"res3_1", 128, true}, {"res3_2", 128, false},
                        {"res4_1", 256, true}, {"res4_2", 256, false}, {"res5_1", 512, true}, {"res6_1", 512, true}};
  for (const Blk& b : blocks) {
    Conv2DShape s;
    s.filters = b.filters; s.kernel = {3, 3}; s.pad = {1, 1};
    NameScope scope(b.name);
    ParallelBatchNormParamOp<Act> blk = b.proj ? spatial_parallel_proj_residual_v2_conv2d<Act>(s, 2, sw, cur, ctx)
                                               : spatial_parallel_residual_v2_conv2d<Act>(s, sw, cur, ctx);
    absorb(net, blk.ops, blk.params, blk.grads, &blk.batch_stats, &blk.fixed_stats);
    cur = blk.ops;
  }
  ParallelBatchNormParamOp<Act> bnf;
  { NameScope scope("bn_final"); bnf = parallel_batch_norm<Act>(512, sw, cur, true, ctx); }
  absorb(net, bnf.ops, bnf.params, bnf.grads, &bnf.batch_stats, &bnf.fixed_stats);
  // strips -> the whole feature map on every rank, global average pool, classifier
  auto full = SpatialAllGather2DOpF::MakeParallel(bnf.ops, ctx);
  Pool2DShape gp;
  gp.pooling = kAveragePool;
  gp.window = {full.at(0)->shape().shape[0], full.at(0)->shape().shape[1]};
  gp.stride = gp.window;
  auto pooled = CudnnPool2DOpF::MakeParallel(gp, full, ctx);
  ParallelParamOp<Act> fc;
  { NameScope scope("fc1"); fc = parallel_linear<Act>(classes, pooled, xavier_init_gen<GPUArray4D<float>>(512, classes), ctx); }
  absorb(net, fc.ops, fc.params, fc.grads);
  net.losses = CudnnSoftmaxNLLLoss2DOpF::MakeParallel(fc.ops, ctx);
  // every rank holds the whole batch: the mean loss, shared out over the R replicas of the head so that the
  // sum over ranks (reduce-scatter of the feature gradient, allreduce of the parameter gradients) is the gradient
  for (auto& l : net.losses) l->set_loss_weight(1.0f / (float)(cfg.batch_size * R));
  net.outputs = fc.ops;
  vector<shared_ptr<Op>> members(net.losses.begin(), net.losses.end());
  net.sink = make_shared<GroupSinkOp>(members);
  for (auto& o : fc.ops) net.output_grad_vars[o->rank()].insert(o->data().grad.var());
  return net;
}

// single-rank twins of the halo_conv / bottleneck helpers for the replicated tail of a net: ordinary zero padding
static vector<ActVar> plain_conv3x3(const char* name, Conv2DShape shape, vector<ActVar> in, BlockVars& vars, shared_ptr<Context> ctx) {
  NameScope scope(name);
  shape.halo_padded_input = true;   // pad -> conv on the padded buffer, without an exchange: every rank holds all rows
  auto pad = HaloPad2DOpF::MakeParallel(shape.pad[0], in, ctx);
  const size_t cin = in.at(0)->shape().shape[2];
  auto conv = parallel_conv2d<Act>(shape, pad, kaiming_init_gen<GPUArray4D<float>>(cin * shape.kernel[0] * shape.kernel[1], shape.filters), false, ctx);
  vars.add(conv);
  return conv.ops;
}
static ParallelBatchNormParamOp<Act> replicated_bottleneck(Conv2DShape shape, size_t bottleneck, size_t stride, bool proj, shared_ptr<bool> sw,
                                                           vector<ActVar> inputs, shared_ptr<Context> ctx) {
  BlockVars vars(inputs.size());
  auto a0 = bn_relu("bn0", inputs.at(0)->shape().shape[2], sw, inputs, vars, ctx);
  vector<ActVar> shortcut = inputs;
  if (proj) shortcut = conv1x1("proj", bottleneck * shape.filters, stride, a0, vars, ctx);
  auto c1 = conv1x1("conv1", shape.filters, 1, a0, vars, ctx);
  auto a1 = bn_relu("bn1", shape.filters, sw, c1, vars, ctx);
  Conv2DShape s2 = shape;
  s2.stride = {stride, stride};
  auto c2 = plain_conv3x3("conv2", s2, a1, vars, ctx);
  auto a2 = bn_relu("bn2", shape.filters, sw, c2, vars, ctx);
  auto c3 = conv1x1("conv3", bottleneck * shape.filters, 1, a2, vars, ctx);
  return vars.finish(parallel_sum<Act>({shortcut, c3}, ctx));
}

template <>
SpatialParallelNet SpatialParallelResNet<float>::MakeParallelResNet50(const ConvNetConfig& cfg, size_t classes, shared_ptr<Context> ctx) {
  vector<ActVar> strips;
  SpatialParallelNet net = begin_net(cfg, ctx, strips, true);
  auto sw = net.batch_norm_use_fixed;
  const size_t R = ranks_of(ctx);
  vector<ActVar> cur = stem(net, cfg, 64, strips, ctx);
  const size_t blocks[4] = {3, 4, 6, 3}, strides[4] = {1, 2, 2, 2};
  bool gathered = R == 1;
  for (int st = 0; st < 4; ++st) {
    Conv2DShape b;
    b.filters = (size_t)64 << st; b.kernel = {3, 3}; b.pad = {1, 1};
    if (!gathered && strides[st] == 2 && (cur.at(0)->shape().shape[1] % 2)) {
      cur = SpatialAllGather2DOpF::MakeParallel(cur, ctx);   // an odd strip cannot be strided: go on replicated
      gathered = true;
    }
    for (size_t i = 0; i < blocks[st]; ++i) {
      NameScope scope("stage" + std::to_string(st + 1) + ".block" + std::to_string(i + 1));
      ParallelBatchNormParamOp<Act> blk;
      if (gathered && R > 1) blk = replicated_bottleneck(b, 4, i == 0 ? strides[st] : 1, i == 0, sw, cur, ctx);
      else blk = i == 0 ? spatial_parallel_proj_bottleneck_residual_v2_conv2d<Act>(b, 4, strides[st], sw, cur, ctx)
                        : spatial_parallel_bottleneck_residual_v2_conv2d<Act>(b, 4, sw, cur, ctx);
      absorb(net, blk.ops, blk.params, blk.grads, &blk.batch_stats, &blk.fixed_stats);
      cur = blk.ops;
    }
  }
  ParallelBatchNormParamOp<Act> bnf;
  { NameScope scope("bn_final"); bnf = parallel_batch_norm<Act>(2048, sw, cur, true, ctx); }
  absorb(net, bnf.ops, bnf.params, bnf.grads, &bnf.batch_stats, &bnf.fixed_stats);
  auto full = (gathered && R > 1) ? bnf.ops : SpatialAllGather2DOpF::MakeParallel(bnf.ops, ctx);
  Pool2DShape gp;
  gp.pooling = kAveragePool;
  gp.window = {full.at(0)->shape().shape[0], full.at(0)->shape().shape[1]};
  gp.stride = gp.window;
  auto pooled = CudnnPool2DOpF::MakeParallel(gp, full, ctx);
  ParallelParamOp<Act> fc;
  { NameScope scope("fc1"); fc = parallel_linear<Act>(classes, pooled, xavier_init_gen<GPUArray4D<float>>(2048, classes), ctx); }
  absorb(net, fc.ops, fc.params, fc.grads);
  net.losses = CudnnSoftmaxNLLLoss2DOpF::MakeParallel(fc.ops, ctx);
  for (auto& l : net.losses) l->set_loss_weight(1.0f / (float)(cfg.batch_size * R));
  net.outputs = fc.ops;
  vector<shared_ptr<Op>> members(net.losses.begin(), net.losses.end());
  net.sink = make_shared<GroupSinkOp>(members);
  for (auto& o : fc.ops) net.output_grad_vars[o->rank()].insert(o->data().grad.var());
  return net;
}


// ------------------------------------------------------------------ the reference's tool-facing builders
static ParallelCategoricalNLLBatchNormLoss<> package_classifier(SpatialParallelNet net, const ConvNetConfig& cfg, shared_ptr<Context> ctx) {
  ParallelCategoricalNLLBatchNormLoss<> out;
  const size_t R = ranks_of(ctx);
  const size_t h = cfg.input_h / R;
  bool first = true;
  for (size_t r = 0; r < R; ++r) {
    if (!local_rank(ctx, r)) continue;
    // one batch of whole NHWC images in 0..255: each rank takes its rows, scaled to 0..1
    net.inputs[r]->set_rows_of_full(cfg.input_h, r * h, true, 1.0f / 255.0f);
    out.inputs.insert(net.inputs[r]->data().val.var());
  }
  for (auto& l : net.losses) {
    // every rank scores the whole batch: the mean over the minibatch, shared out over the R copies of the head
    l->set_loss_weight(1.0f / (float)((cfg.minibatch_size ? cfg.minibatch_size : cfg.batch_size) * R));
    l->set_replica(!first);
    out.labels.insert(l->label_var());
    if (first) {
      out.losses.insert(l->loss_var());
      out.loss = l;
      for (auto& o : net.outputs)
        if (o->rank() == l->rank()) out.logits.insert(o->data().val.var());
    }
    first = false;
  }
  out.batch_norm_use_fixed = net.batch_norm_use_fixed;
  // `op` is what a tool initialises from (op->init): the root, so that every rank's variables are reached
  out.sum_loss = net.sink;
  out.op = net.sink;
  out.dev_params = net.dev_params; out.dev_grads = net.dev_grads;
  out.dev_batch_stats = net.dev_batch_stats; out.dev_fixed_stats = net.dev_fixed_stats;
  out.net = net;
  return out;
}
template <>
ParallelCategoricalNLLBatchNormLoss<> ResNet<float>::MakeParallelResNet18(const ConvNetConfig& cfg, shared_ptr<Context> ctx) {
  return package_classifier(SpatialParallelResNet<float>::MakeParallelResNet18(cfg, 1000, ctx), cfg, ctx);
}
template <>
ParallelCategoricalNLLBatchNormLoss<> ResNet<float>::MakeParallelResNet50(const ConvNetConfig& cfg, shared_ptr<Context> ctx) {
  return package_classifier(SpatialParallelResNet<float>::MakeParallelResNet50(cfg, 1000, ctx), cfg, ctx);
}

}  // namespace arraydiff
