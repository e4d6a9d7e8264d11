// Model builders of the spatially parallel path.  Same entry points as the reference's
// include/arraydiff/zoo.hh:61-190 for this path (conv2d / parallel_conv2d, the spatial_parallel_*
// residual blocks); bodies compose the operators of op.hh per rank, in the same order on every rank
// so that flat parameter buffers line up (reference include/arraydiff/optimize.hh:323-333).
#ifndef ARRAYDIFF_ZOO_HH
#define ARRAYDIFF_ZOO_HH

#include "arraydiff/op.hh"

namespace arraydiff {

template <typename V> struct ParamOp { shared_ptr<Var<V>> op; VarIdSet params, grads; };
template <typename V> struct ParallelParamOp { vector<shared_ptr<Var<V>>> ops; vector<VarIdSet> params, grads; };
template <typename V> struct BatchNormParamOp { shared_ptr<Var<V>> op; VarIdSet params, grads, batch_stats, fixed_stats; };
template <typename V> struct ParallelBatchNormParamOp {
  vector<shared_ptr<Var<V>>> ops;
  vector<VarIdSet> params, grads, batch_stats, fixed_stats;
};

typedef IOOp<GPUArray4D<float>>::InitFn KernelInitFn;
// normal(0, sqrt(2 / fan_in)), drawn on the host from the shared generator (reference src/op.cc:362-408)
template <typename A> typename IOOp<A>::InitFn kaiming_init_gen(size_t fan_in, size_t fan_out);
// uniform(+-sqrt(6 / (fan_in + fan_out)))   (reference src/op.cc:362-408)
template <typename A> typename IOOp<A>::InitFn xavier_init_gen(size_t fan_in, size_t fan_out);
template <typename A> typename IOOp<A>::InitFn zeros_init_gen();

template <typename V> ParamOp<V> conv2d(Conv2DShape shape, shared_ptr<Var<V>> input, KernelInitFn kernel_init, bool enable_bias, shared_ptr<Context> ctx);
template <typename V> ParallelParamOp<V> parallel_conv2d(Conv2DShape shape, vector<shared_ptr<Var<V>>> inputs, KernelInitFn kernel_init, bool enable_bias, shared_ptr<Context> ctx);
// fully connected layer with bias on [batch][features] activations, one replica per rank (reference src/zoo.cc:62-90)
template <typename V> ParamOp<V> linear(size_t filters, shared_ptr<Var<V>> input, KernelInitFn kernel_init, shared_ptr<Context> ctx);
template <typename V> ParallelParamOp<V> parallel_linear(size_t filters, vector<shared_ptr<Var<V>>> inputs, KernelInitFn kernel_init, shared_ptr<Context> ctx);
template <typename V> vector<shared_ptr<Var<V>>> parallel_relu(vector<shared_ptr<Var<V>>> inputs, shared_ptr<Context> ctx);
template <typename V> vector<shared_ptr<Var<V>>> parallel_sum(vector<vector<shared_ptr<Var<V>>>> inputs, shared_ptr<Context> ctx);
// batch norm per rank, optionally with the following ReLU folded in
template <typename V> ParallelBatchNormParamOp<V> parallel_batch_norm(size_t channels, shared_ptr<bool> switch_var, vector<shared_ptr<Var<V>>> inputs, bool fuse_relu, shared_ptr<Context> ctx);

template <typename V> ParallelBatchNormParamOp<V> spatial_parallel_residual_v2_conv2d(Conv2DShape shape, shared_ptr<bool> switch_var, vector<shared_ptr<Var<V>>> inputs, shared_ptr<Context> ctx);
template <typename V> ParallelBatchNormParamOp<V> spatial_parallel_proj_residual_v2_conv2d(Conv2DShape shape, size_t stride, shared_ptr<bool> switch_var, vector<shared_ptr<Var<V>>> inputs, shared_ptr<Context> ctx);
template <typename V> ParallelBatchNormParamOp<V> spatial_parallel_bottleneck_residual_v2_conv2d(Conv2DShape shape, size_t bottleneck, shared_ptr<bool> switch_var, vector<shared_ptr<Var<V>>> inputs, shared_ptr<Context> ctx);
template <typename V> ParallelBatchNormParamOp<V> spatial_parallel_proj_bottleneck_residual_v2_conv2d(Conv2DShape shape, size_t bottleneck, size_t stride, shared_ptr<bool> switch_var, vector<shared_ptr<Var<V>>> inputs, shared_ptr<Context> ctx);

class ConvNetConfig {
public:
  size_t input_c = 3, input_w = 0, input_h = 0, batch_size = 1, minibatch_size = 1;
};

// A spatially partitioned feature extractor: per-rank inputs (the full image, scattered into
// H-strips inside the graph), per-rank outputs (strips), and the per-rank variable sets.
// Depth / width of the dilated segmentation net: channels of stage s are base << s (x4 at the block
// outputs); blocks {3,4,6,3} with base 64 is ResNet-50.
struct SegNetConfig {
  size_t base = 64;
  size_t blocks[4] = {3, 4, 6, 3};
  size_t classes = 19;
};

struct SpatialParallelNet {
  shared_ptr<bool> batch_norm_use_fixed;
  vector<shared_ptr<IOOp<Act>>> inputs;
  vector<ActVar> outputs;
  vector<shared_ptr<CudnnSoftmaxNLLLoss2DOpF>> losses;   // per-rank loss sinks (nets that end in a loss)
  shared_ptr<Op> sink;          // GroupSinkOp over all outputs (or losses): walk from here
  VarIdSet input_vars;
  vector<VarIdSet> output_grad_vars;
  vector<VarIdSet> dev_params, dev_grads, dev_batch_stats, dev_fixed_stats;
};

// What the reference's builders hand to a training tool (include/arraydiff/zoo.hh:140-158): the graph's root, the
// variable sets a tool loads and stores through (one batch of inputs and labels in, logits and per-image losses out),
// and the per-rank parameter / gradient / statistics sets the optimizer walks.  The three class parameters of the
// reference (array types of logits, losses and the summed loss) are kept for spelling only: every variable here is
// reached through shared_ptr<Op>.
template <typename Logit = Act, typename Loss = Act, typename SumLoss = Act>
class ParallelCategoricalNLLBatchNormLoss {
public:
  shared_ptr<bool> batch_norm_use_fixed;
  shared_ptr<Op> op;          // where a tool starts op->init from: the root, so that every rank's variables are drawn
  shared_ptr<Op> loss;        // rank 0's per-image loss
  shared_ptr<Op> sum_loss;    // the root of the whole graph: persist / load_val / gradient / store_val start here
  VarIdSet inputs;            // every rank's input strip: together one batch of whole images
  VarIdSet labels;
  VarIdSet logits;
  VarIdSet losses;
  vector<VarIdSet> dev_params;
  vector<VarIdSet> dev_grads;
  vector<VarIdSet> dev_batch_stats;
  vector<VarIdSet> dev_fixed_stats;
  SpatialParallelNet net;     // the underlying per-rank view
};

// The reference's entry points for its training tools (include/arraydiff/zoo.hh:175-183, src/zoo.cc:1475-1909,
// :2200-2484): 1000 classes; host images are read as [image][row][column][channel] floats in 0..255 and scaled by
// 1/255 on load (the reference's TransposeNHWCToNCHWOp + ScaleOp in front of the net), each rank taking its rows; the
// loss is the mean over config.minibatch_size images.
template <typename T>
class ResNet {
public:
  static ParallelCategoricalNLLBatchNormLoss<> MakeParallelResNet18(const ConvNetConfig& config, shared_ptr<Context> ctx);
  static ParallelCategoricalNLLBatchNormLoss<> MakeParallelResNet50(const ConvNetConfig& config, shared_ptr<Context> ctx);
};

template <typename T>
class SpatialParallelResNet {
public:
  // One 3x3 convolution (stride 1, pad 1, bias) over H-strips: scatter -> halo pad -> halo exchange ->
  // conv.  The plumbing case of the partitioned path.
  // `first_pad` != 1: the strip is first framed with that halo width and re-framed to 1 (HaloRepad2DOp).
  static SpatialParallelNet MakeConv3x3(const ConvNetConfig& config, size_t filters, shared_ptr<Context> ctx, size_t first_pad = 1);
  // The same layer between the reference's collective operators: BroadcastOp -> SpatialScatter2DOp -> pad / exchange /
  // conv -> SpatialGather2DOp -> AllreduceOp -> ReduceOp.  One output on rank 0: R times the convolution.
  static SpatialParallelNet MakeConv3x3Collectives(const ConvNetConfig& config, size_t filters, shared_ptr<Context> ctx);
  // ResNet-50 stem + stage 1: 7x7/2 conv to 64 channels, BN, ReLU, 3x3/2 max pool, then three
  // pre-activation bottleneck blocks (64-64-256), the first with a 1x1 projection.
  static SpatialParallelNet MakeStemStage1(const ConvNetConfig& config, shared_ptr<Context> ctx);
  // The reference's spatially parallel classifier (ResNet<float>::MakeParallelResNet18, src/zoo.cc:1475-1909): 7x7
  // conv with bias at stride 1, 3x3/2 max pool, basic pre-activation residual blocks 64,64 / 128,128 / 256,256 /
  // 512 / 512 (each first block of a width strided by 2 with a projection), BN + ReLU, re-assembly of the strips
  // on every rank, global average pool, linear classifier, softmax NLL.  Every rank computes the (tiny) head
  // on the whole batch; labels go to every net.losses[r]->load_labels.
  static SpatialParallelNet MakeParallelResNet18(const ConvNetConfig& config, size_t classes, shared_ptr<Context> ctx);
  // ResNet-50 classifier over H-strips (the reference's MakeParallelResNet50 entry, src/zoo.cc:2200-2484, there an
  // 18-layer body; here the bottleneck stages {3,4,6,3} built from spatial_parallel_*bottleneck* blocks): stem,
  // max pool, stages strided 1,2,2,2, BN + ReLU, all-gather, global average pool, linear, softmax NLL.  A strided
  // stage needs an even strip height; when a stage would meet an odd one (224 rows over 2 strips reach 7 rows per
  // strip in front of stage 4) the strips are re-assembled in front of it and the rest runs replicated per rank.
  static SpatialParallelNet MakeParallelResNet50(const ConvNetConfig& config, size_t classes, shared_ptr<Context> ctx);
  // Dilated ResNet-50 segmentation net at output stride 8 with a bilinear x8 head and per-pixel loss
  // (the 1024x2048, 19-class configuration); labels go to net.losses[r]->load_labels.
  static SpatialParallelNet MakeSegNet50(const ConvNetConfig& config, const SegNetConfig& seg, shared_ptr<Context> ctx);
};

}  // namespace arraydiff
#endif
