// The op-graph runtime and the operators of the spatially parallel convolution path.
// Same model as the reference's include/arraydiff/op.hh / src/op.cc:
//   * identity counters NodeId / EpochId / TxnId / VarId are thread-local, monotonically increasing
//     (reference src/op.cc:77-110);
//   * a graph walk visits every node once per epoch: _push recurses into the inputs on the first
//     push and then applies, _pop applies once every consumer has popped and then pops the inputs in
//     reverse (reference op.hh:1872-1892, OperatorStack src/op.cc:112-146); forward = push-apply,
//     backward = pop-apply (src/op.cc:214-234);
//   * TxnVar<V> is a lazily allocated buffer stamped with the transaction that wrote it:
//     overwrite / accumulate / get / get_excl / get_mut / rollover (reference op.hh:188-489);
//   * every _backward ADDS into its inputs' gradients after a once-per-transaction zero fill;
//   * load_val / store_val / store_grad walk the graph and move only IOOp data, each variable once
//     (reference op.hh:152-163, 831-861); variables are laid out in operator creation order, which is
//     the same on every rank, so that flat buffers of different ranks line up element by element.
// Operator classes keep the reference's names (the Cudnn prefix included) although no cuDNN is
// called: every body is a call into the arraydiff_b200 C ABI.
#ifndef ARRAYDIFF_OP_HH
#define ARRAYDIFF_OP_HH

#include <any>
#include <cassert>
#include <functional>
#include <memory>
#include <optional>
#include <random>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "arraydiff/array_gpu.hh"
#include "arraydiff/context.hh"
#include "arraydiff/slice.hh"
#include "arraydiff/spatial.hh"

namespace arraydiff {

using std::any;
using std::function;
using std::make_shared;
using std::shared_ptr;
using std::string;
using std::vector;

class NodeId { public: NodeId(); uint64_t raw_id() const { return id_; } private: uint64_t id_; };
class EpochId { public: EpochId(); uint64_t raw_id() const { return id_; } private: uint64_t id_; };
class TxnId { public: TxnId(); uint64_t raw_id() const { return id_; } private: uint64_t id_; };
enum VarKind { VAR_KIND_VAL, VAR_KIND_GRAD };
class VarId {
public:
  VarId();
  explicit VarId(VarKind k);
  uint64_t raw_id() const { return id_; }
  VarKind kind() const { return kind_; }
private:
  uint64_t id_;
  VarKind kind_;
};

class VarIdSet {
public:
  static VarIdSet Singleton(VarId v) { VarIdSet s; s.insert(v); return s; }
  VarIdSet() : locked_(false) {}
  size_t size() const { return vars_.size(); }
  void lock() { assert(!locked_); mask_.clear(); locked_ = true; }
  void unlock() { assert(locked_); locked_ = false; mask_.clear(); }
  bool contains(VarId v) const { return vars_.count(v.raw_id()) > 0; }
  void insert(VarId v) { assert(!locked_); vars_.insert(v.raw_id()); }
  void insert_all(const VarIdSet& o) { assert(!locked_); vars_.insert(o.vars_.begin(), o.vars_.end()); }
  // true exactly once per locked walk for a member variable
  bool mask(VarId v) {
    assert(locked_);
    if (!vars_.count(v.raw_id())) return false;
    return mask_.insert(v.raw_id()).second;
  }
private:
  bool locked_;
  std::unordered_set<uint64_t> vars_, mask_;
};

template <typename V>
struct TxnVarBuf {
  std::optional<uint64_t> curr_txn;
  bool rollover = false;
  std::unordered_set<uint64_t> writers;
  std::optional<V> buffer;
  function<V()> alloc;
  VarId id;
};

template <typename V>
class TxnVar {
public:
  TxnVar() {}
  TxnVar(VarKind kind, function<V()> alloc) : buf_(make_shared<TxnVarBuf<V>>()) { buf_->alloc = alloc; buf_->id = VarId(kind); }
  VarId var() const { return buf_->id; }
  bool allocated() const { return buf_ && buf_->buffer.has_value(); }
  // true if `node` should (re)produce the value in this transaction
  bool overwrite(TxnId txn, NodeId node) {
    ensure();
    if (!buf_->curr_txn || *buf_->curr_txn != txn.raw_id()) {
      buf_->curr_txn = txn.raw_id(); buf_->rollover = false; buf_->writers.clear();
      buf_->writers.insert(node.raw_id());
      return true;
    }
    if (buf_->rollover) return false;
    return buf_->writers.insert(node.raw_id()).second;
  }
  // true if `node` has not yet added its contribution in this transaction; init runs once per
  // transaction unless the variable was rolled over
  bool accumulate(TxnId txn, NodeId node, function<void(V*)> init) {
    ensure();
    if (!buf_->curr_txn || *buf_->curr_txn != txn.raw_id()) {
      buf_->curr_txn = txn.raw_id(); buf_->rollover = false; buf_->writers.clear();
      if (init) init(&*buf_->buffer);
    }
    return buf_->writers.insert(node.raw_id()).second;
  }
  // accumulate() for a contributor that may write the WHOLE buffer: returns 0 if `node` has already
  // contributed in this transaction, 2 if it is the first contributor and covers(buffer) holds -- it
  // then OVERWRITES (no zero fill, no read of the old value) -- and 1 (add; init has run if needed) otherwise.
  int accumulate_full(TxnId txn, NodeId node, function<bool(V&)> covers, function<void(V*)> init) {
    ensure();
    if (!buf_->curr_txn || *buf_->curr_txn != txn.raw_id()) {
      buf_->curr_txn = txn.raw_id(); buf_->rollover = false; buf_->writers.clear();
      buf_->writers.insert(node.raw_id());
      if (covers && covers(*buf_->buffer)) return 2;
      if (init) init(&*buf_->buffer);
      return 1;
    }
    return buf_->writers.insert(node.raw_id()).second ? 1 : 0;
  }
  V& get(TxnId txn, NodeId) { assert(buf_->buffer && buf_->curr_txn && *buf_->curr_txn == txn.raw_id()); return *buf_->buffer; }
  V& get_excl(TxnId txn, NodeId n) { return get(txn, n); }
  V& get_mut(TxnId txn, NodeId n) { return get(txn, n); }
  V& raw() { ensure(); return *buf_->buffer; }   // no transaction check (optimizer / tests)
  bool written_in(TxnId txn) const { return buf_->curr_txn && *buf_->curr_txn == txn.raw_id(); }
  void rollover(TxnId txn, VarIdSet& vars) {
    if (!vars.contains(buf_->id)) return;
    ensure();
    buf_->curr_txn = txn.raw_id(); buf_->rollover = true; buf_->writers.clear();
  }
  void stamp(TxnId txn) { ensure(); buf_->curr_txn = txn.raw_id(); buf_->rollover = true; buf_->writers.clear(); }
private:
  void ensure() { if (!buf_->buffer) buf_->buffer = buf_->alloc(); }
  shared_ptr<TxnVarBuf<V>> buf_;
};

template <typename V>
struct VarData {
  TxnVar<V> val, grad;
  VarData() {}
  explicit VarData(function<V()> alloc) : val(VAR_KIND_VAL, alloc), grad(VAR_KIND_GRAD, alloc) {}
};

class OperatorStack {
public:
  size_t push(EpochId e);
  size_t degree(EpochId e);
  size_t pop(EpochId e);
private:
  struct Entry { uint64_t epoch; size_t push_count, pop_count; };
  vector<Entry> entries_;
};

class Op {
public:
  Op() {}
  virtual ~Op() {}
  NodeId id() const { return node_id_; }

  virtual void _push(EpochId epoch, function<void(Op*)> apply);
  virtual void _pop(EpochId epoch, function<void(Op*)> apply);
  virtual size_t _load_val(TxnId, VarIdSet&, size_t offset, any*) { return offset; }
  virtual size_t _load_grad(TxnId, VarIdSet&, size_t offset, any*) { return offset; }
  virtual size_t _store_val(TxnId, VarIdSet&, size_t offset, any*) { return offset; }
  virtual size_t _store_grad(TxnId, VarIdSet&, size_t offset, any*) { return offset; }
  virtual void _init(TxnId, std::mt19937_64*) {}
  virtual void _persist(TxnId, VarIdSet&) {}
  virtual void _set_grad_sink(TxnId) { assert(0 && "not a scalar sink"); }
  virtual void _forward(TxnId txn) = 0;
  virtual void _backward(TxnId txn) = 0;
  virtual string _debug_op_label() { return "Op"; }

  size_t load_val(TxnId txn, VarIdSet& vars, size_t offset, any* reader);
  size_t load_grad(TxnId txn, VarIdSet& vars, size_t offset, any* reader);
  size_t store_val(TxnId txn, VarIdSet& vars, size_t offset, any* writer);
  size_t store_grad(TxnId txn, VarIdSet& vars, size_t offset, any* writer);
  void init(TxnId txn, std::mt19937_64* rng);
  void persist(TxnId txn, VarIdSet& vars);
  void eval(TxnId txn);                 // forward walk
  void gradient(TxnId txn);             // forward, unit gradient at this (scalar) sink, backward
  void backward(TxnId txn);             // backward walk only: the sink's gradient was loaded with load_grad

protected:
  vector<shared_ptr<Op>> inputs_;
  NodeId node_id_;
  OperatorStack stack_;
};

template <typename V>
class Var : public virtual Op {
public:
  virtual typename V::Shape shape() = 0;
  virtual size_t batch_shape() = 0;
  virtual VarData<V> data() = 0;
  virtual vector<VarId> vars() { auto d = data(); return {d.val.var(), d.grad.var()}; }
  virtual size_t rank() const { return 0; }
};

typedef GPUBatchArray3D<float> Act;
typedef shared_ptr<Var<Act>> ActVar;

// ---------------------------------------------------------------- shapes (reference op.hh:1799-1810, 2912-2925)
class Conv2DShape {
public:
  Conv2DShape() : filters(0), axes({0, 1}), kernel({1, 1}), dilate({1, 1}), stride({1, 1}), pad({0, 0}),
                  halo_padded_input(false), enable_hmma(false) {}
  size_t filters;
  std::array<size_t, 2> axes, kernel, dilate, stride, pad;   // {w-axis, h-axis} pairs
  bool halo_padded_input;
  bool enable_hmma;
  Shape3D calculate_output_shape(Shape3D in) const;
};
enum PoolKind { kMaxPool, kAveragePool };
class Pool2DShape {
public:
  Pool2DShape() : pooling(kMaxPool), axes({0, 1}), window({1, 1}), stride({1, 1}), pad({0, 0}), halo_padded_input(false) {}
  PoolKind pooling;
  std::array<size_t, 2> axes, window, stride, pad;
  bool halo_padded_input;
  Shape3D calculate_output_shape(Shape3D in) const;
};

// ---------------------------------------------------------------- IO variables (reference IOOp / SrcOp, op.hh:831-1017)
template <typename A> struct IOTraits;

// Optional naming of parameters, so that a flat parameter buffer can be taken apart again:
// builders open a NameScope per layer, IOOps remember the scope they were created in, and a
// store_val walk whose writer holds a ParamManifest* records (name, offset, size) instead of copying.
struct ParamManifestEntry { string name; size_t offset, size; };
typedef vector<ParamManifestEntry> ParamManifest;
class NameScope {
public:
  explicit NameScope(const string& name);
  ~NameScope();
  static string current();
};

template <typename A>
class IOOp : public Var<A> {
public:
  typedef function<void(A*, std::mt19937_64*, shared_ptr<Context>)> InitFn;
  static shared_ptr<IOOp<A>> Make(typename A::Shape dim, size_t batch, InitFn init, size_t rank, shared_ptr<Context> ctx) {
    return make_shared<IOOp<A>>(dim, batch, init, rank, ctx);
  }
  IOOp(typename A::Shape dim, size_t batch, InitFn init, size_t rank, shared_ptr<Context> ctx);
  typename A::Shape shape() override { return dim_; }
  size_t batch_shape() override { return batch_; }
  VarData<A> data() override { return data_; }
  size_t rank() const override { return rank_; }
  void _forward(TxnId) override {}
  void _backward(TxnId) override {}
  void _init(TxnId txn, std::mt19937_64* rng) override;
  void _persist(TxnId txn, VarIdSet& vars) override { data_.val.rollover(txn, vars); }
  size_t _load_val(TxnId txn, VarIdSet& vars, size_t offset, any* reader) override;
  size_t _load_grad(TxnId txn, VarIdSet& vars, size_t offset, any* reader) override;
  size_t _store_val(TxnId txn, VarIdSet& vars, size_t offset, any* writer) override;
  size_t _store_grad(TxnId txn, VarIdSet& vars, size_t offset, any* writer) override;
  string _debug_op_label() override { return "IOOp"; }
  void set_name(const string& n) { name_ = n; }
  const string& name() const { return name_; }
  // An activation input that holds rows [row0, row0 + h) of a batch of full_h-row images: a reader that carries the
  // WHOLE batch (float* / Slice<float>) is then cut on load -- every rank takes its rows of the same host buffer and
  // the flat offset advances by the strip's share, so that all ranks' inputs together account for the batch once.
  // nhwc: the host batch is [image][row][column][channel] (the reference's raw input, Shape3D(3, w, h), src/zoo.cc:1503);
  // host_scale multiplies every element on the way in (its ScaleOp(1/255), src/zoo.cc:1515).
  void set_rows_of_full(size_t full_h, size_t row0, bool nhwc, float host_scale) {
    full_h_ = full_h; row0_ = row0; host_nhwc_ = nhwc; host_scale_ = host_scale;
  }
private:
  size_t full_h_ = 0, row0_ = 0;
  bool host_nhwc_ = false;
  float host_scale_ = 1.0f;
  string name_;
  typename A::Shape dim_;
  size_t batch_, rank_;
  InitFn init_;
  shared_ptr<Context> ctx_;
  VarData<A> data_;
};
template <typename A> using SrcOp = IOOp<A>;
// A reader for activations that lets every rank take only its rows of a full host image (packed NCHW fp32).
struct HostRows { const float* base; size_t full_h, row0; };

// Common base of activation operators of one rank.
class ActOp : public Var<Act> {
public:
  ActOp(size_t rank, shared_ptr<Context> ctx) : rank_(rank), ctx_(ctx) {}
  Shape3D shape() override { return dim_; }
  size_t batch_shape() override { return batch_; }
  VarData<Act> data() override { return y_; }
  size_t rank() const override { return rank_; }
  void _persist(TxnId, VarIdSet&) override {}
  // Any activation can be read back, and its gradient set or read, as packed NCHW fp32 of the
  // interior: that is how a caller supplies an upstream gradient or inspects a result.
  size_t _load_grad(TxnId txn, VarIdSet& vars, size_t offset, any* reader) override;
  size_t _store_val(TxnId txn, VarIdSet& vars, size_t offset, any* writer) override;
  size_t _store_grad(TxnId txn, VarIdSet& vars, size_t offset, any* writer) override;
protected:
  GPUContext* gpu();
  MultiGPUContext* mgpu();
  void alloc_output(Shape3D dim, size_t pad_w, size_t pad_h, size_t batch);
  size_t rank_;
  shared_ptr<Context> ctx_;
  Shape3D dim_;
  size_t batch_ = 0;
  VarData<Act> y_;
};

// ---------------------------------------------------------------- spatial operators
// y_r = x[:, :, r*h:(r+1)*h, :]   (reference src/op.cc:2383-2468)
class SpatialScatter2DOpF : public ActOp {
public:
  static vector<ActVar> MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx);
  SpatialScatter2DOpF(size_t rank, size_t num_ranks, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  ActVar x_;
  size_t num_ranks_;
};
// places the strip into a zeroed full-height tensor (reference src/op.cc:2470-2553)
class SpatialGather2DOpF : public ActOp {
public:
  static vector<ActVar> MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx);
  SpatialGather2DOpF(size_t rank, size_t num_ranks, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  ActVar x_;
  size_t num_ranks_;
};
// interior -> zeroed padded buffer; backward dx += interior(dy)   (reference src/op.cc:2555-2712)
class HaloPad2DOpF : public ActOp {
public:
  static vector<ActVar> MakeParallel(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx);
  HaloPad2DOpF(size_t halo_pad, size_t rank, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  size_t halo_pad() const { return pad_; }
private:
  ActVar x_;
  size_t pad_;
};
// padded -> interior (reference src/op.cc:2714-2870)
class HaloUnpad2DOpF : public ActOp {
public:
  static vector<ActVar> MakeParallel(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx);
  HaloUnpad2DOpF(size_t halo_pad, size_t rank, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  ActVar x_;
  size_t pad_;
};
// padded(p_in) -> padded(p_out); the reference defines only the forward (src/op.cc:2872-2960),
// here the backward is the matching interior accumulate.
class HaloRepad2DOpF : public ActOp {
public:
  static vector<ActVar> MakeParallel(size_t src_pad, size_t dst_pad, vector<ActVar> inputs, shared_ptr<Context> ctx);
  HaloRepad2DOpF(size_t src_pad, size_t dst_pad, size_t rank, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  ActVar x_;
  size_t src_pad_, dst_pad_;
};

// One shared op over all ranks; mutates the padded buffers in place.  Outputs are aliases of the
// inputs' data (reference src/op.cc:2962-3052, op.hh:2648-2660).
class HaloExch2DOpF : public virtual Op {
public:
  static vector<ActVar> MakeParallel(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx);
  HaloExch2DOpF(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "HaloExch2DOp"; }
private:
  void run(TxnId txn, bool reduce);
  std::optional<uint64_t> done_fwd_, done_bwd_;
  size_t pad_;
  vector<ActVar> xs_;
  shared_ptr<Context> ctx_;
};
// per-rank alias of a shared op's result
class AliasOpF : public Var<Act> {
public:
  AliasOpF(shared_ptr<Op> shared, ActVar aliased) : aliased_(aliased) { inputs_.push_back(shared); }
  Shape3D shape() override { return aliased_->shape(); }
  size_t batch_shape() override { return aliased_->batch_shape(); }
  VarData<Act> data() override { return aliased_->data(); }
  size_t rank() const override { return aliased_->rank(); }
  void _forward(TxnId) override {}
  void _backward(TxnId) override {}
  ActVar aliased() { return aliased_; }
private:
  ActVar aliased_;
};

// ---------------------------------------------------------------- dense operators
class CudnnConv2DOpF : public ActOp {
public:
  typedef GPUArray4D<float> Kernel;
  typedef GPUArray1D<float> Bias;
  static shared_ptr<CudnnConv2DOpF> Make(Conv2DShape shape, ActVar x, shared_ptr<Var<Kernel>> kernel,
                                         shared_ptr<Var<Bias>> bias, shared_ptr<Context> ctx);
  CudnnConv2DOpF(Conv2DShape shape, ActVar x, shared_ptr<Var<Kernel>> kernel, shared_ptr<Var<Bias>> bias,
                 shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "CudnnConv2DOp"; }
private:
  void fill_args(ad_conv2d_args& a, Act& x);
  void refresh_filter(TxnId txn, cudaStream_t s);
  Conv2DShape shape_;
  ActVar x_;
  shared_ptr<Var<Kernel>> kernel_;
  shared_ptr<Var<Bias>> bias_;
  Shape3D in_dim_;
  // tensor-core path: bf16 KRSC copy of the filter, fp32 KRSC gradient staging, im2col matrix (stem)
  void* w_bf16_ = nullptr;
  float* dw_krsc_ = nullptr;
  void* im2col_ = nullptr;
  size_t ck_ = 0;       // channels the tensor-core kernel reduces over per tap (padded)
  bool use_im2col_ = false;
  std::optional<uint64_t> filter_txn_;
};

class CudnnPool2DOpF : public ActOp {
public:
  static shared_ptr<CudnnPool2DOpF> Make(Pool2DShape shape, ActVar x, shared_ptr<Context> ctx);
  static vector<ActVar> MakeParallel(Pool2DShape shape, vector<ActVar> inputs, shared_ptr<Context> ctx);
  CudnnPool2DOpF(Pool2DShape shape, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  Pool2DShape shape_;
  ActVar x_;
};

// Spatial batch norm with batch statistics of THIS rank's strip (the reference's behaviour, src/op.cc:3988-4003).
// When the net's switch variable is set the forward pass normalises with the fixed (running) statistics instead
// (src/op.cc:3964-3978); like the reference, that mode has no backward pass.  Statistics over all ranks' strips
// together are available at the C ABI (ad_bn_partial_stats / ad_bn_finalize_apply), not through this operator.
class CudnnBatchNorm2DOpF : public ActOp {
public:
  typedef GPUArray1D<float> Stat;
  struct Parts {
    shared_ptr<CudnnBatchNorm2DOpF> op;
    shared_ptr<IOOp<Stat>> scale, shift, batch_mean, batch_variance, fixed_mean, fixed_variance;
  };
  static Parts Make(size_t channels, shared_ptr<bool> switch_var, ActVar x, shared_ptr<Context> ctx);
  CudnnBatchNorm2DOpF(shared_ptr<bool> switch_var, ActVar x, Parts* parts, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  void fuse_relu() { relu_ = true; }
  bool relu_fused() const { return relu_; }
private:
  shared_ptr<bool> switch_var_;
  ActVar x_;
  shared_ptr<IOOp<Stat>> scale_, shift_, batch_mean_, batch_variance_, fixed_mean_, fixed_variance_;
  float *save_mean_ = nullptr, *save_invstd_ = nullptr;
  bool relu_ = false;
};

enum ActivationKind { kReluAct };
class CudnnActivationOpF : public ActOp {
public:
  static ActVar Make(ActivationKind, ActVar x, shared_ptr<Context> ctx);
  CudnnActivationOpF(ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  ActVar x_;
};

class SumJoin {};
// y = sum_i x_i ; dx_i += dy  (reference src/op.cc:630-867)
class SumJoinOpF : public ActOp {
public:
  static ActVar Make(vector<ActVar> xs, shared_ptr<Context> ctx);
  SumJoinOpF(vector<ActVar> xs, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  vector<ActVar> xs_;
};

// Re-assembly of the strips on every rank: y_r = concat_q x_q along H.  The reference builds it from
// SpatialGather2DOp (strip into a zeroed full tensor) followed by AllreduceOp (src/zoo.cc:1841-1842), which
// moves R times the bytes; here every rank pulls its peers' strips (peer loads inside one process, peer
// loads ordered by flag words between processes).  Backward is the matching reduce-scatter:
// dx_r (+)= sum_q dy_q[rows of strip r], peers in rank order.
class SpatialAllGather2DOpF;
// one rank's gathered tensor: owns the buffers, the shared operator fills them
class AllGatherOutF : public ActOp {
public:
  AllGatherOutF(shared_ptr<SpatialAllGather2DOpF> shared, ActVar strip, size_t num_ranks, shared_ptr<Context> ctx);
  void _forward(TxnId) override {}
  void _backward(TxnId) override {}
};
// One operator over all ranks, like HaloExch2DOp: its backward runs once every rank's consumer has
// delivered the gradient of its gathered tensor.
class SpatialAllGather2DOpF : public virtual Op {
public:
  static vector<ActVar> MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx);
  SpatialAllGather2DOpF(vector<ActVar> inputs, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "SpatialAllGather2DOp"; }
private:
  void wait_peers(size_t rank, cudaStream_t s);
  std::optional<uint64_t> done_fwd_, done_bwd_;
  vector<ActVar> xs_;
  vector<AllGatherOutF*> outs_;      // same order as xs_; owned by the graph (they hold this operator as their input)
  shared_ptr<Context> ctx_;
  size_t num_ranks_;
};

// ---------------------------------------------------------------- collectives as graph operators
// The reference's BroadcastOp (src/op.cc:1854-1966), AllreduceOp (:2284-2381) and ReduceOp (:1968-2174): one operator
// shared by all ranks, results exposed per rank.  They serve graphs written the reference's way (broadcast the image,
// cut strips inside the graph; gather strips into zeroed full tensors and all-reduce them; reduce the replicas'
// logits to rank 0) inside ONE process, where ranks reach each other's buffers directly and are ordered by CUDA
// events; the builders in zoo.hh use scatter-on-load and SpatialAllGather2DOp instead, which also work between
// processes.  Sums run in rank order on every rank (same bits everywhere).  The backward passes ACCUMULATE into the
// inputs' gradients (the reference overwrites them: FIXMEs at src/op.cc:1938, :2366, and passes a reduction operator
// where a root rank belongs at :2057-2063).
class CollectiveOutF : public ActOp {     // one rank's result buffer of a shared collective
public:
  CollectiveOutF(shared_ptr<Op> shared, ActVar like, size_t rank, shared_ptr<Context> ctx);
  void _forward(TxnId) override {}
  void _backward(TxnId) override {}
};
class BroadcastOpF : public virtual Op {
public:
  // y_r = x (which lives on `root`) for every rank r
  static vector<ActVar> MakeParallel(size_t root, ActVar x, shared_ptr<Context> ctx);
  BroadcastOpF(size_t root, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "BroadcastOp"; }
private:
  std::optional<uint64_t> done_fwd_, done_bwd_;
  size_t root_;
  ActVar x_;
  vector<CollectiveOutF*> outs_;
  shared_ptr<Context> ctx_;
};
class AllreduceOpF : public virtual Op {
public:
  // y_r = sum_q x_q on every rank
  static vector<ActVar> MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx);
  AllreduceOpF(vector<ActVar> inputs, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "AllreduceOp"; }
private:
  std::optional<uint64_t> done_fwd_, done_bwd_;
  vector<ActVar> xs_;
  vector<CollectiveOutF*> outs_;
  shared_ptr<Context> ctx_;
};
class ReduceOpF : public virtual Op {
public:
  // y = sum_q x_q on `root`
  static ActVar MakeParallel(size_t root, vector<ActVar> inputs, shared_ptr<Context> ctx);
  ReduceOpF(size_t root, vector<ActVar> inputs, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "ReduceOp"; }
private:
  std::optional<uint64_t> done_fwd_, done_bwd_;
  size_t root_;
  vector<ActVar> xs_;
  CollectiveOutF* out_ = nullptr;
  shared_ptr<Context> ctx_;
};

// y = x w^T + b on [batch][features] activations (1 x 1 spatial extent), w Shape4D(1,1,in,out) = [out][in] in
// memory.  The reference's CublasLinearOp (src/op.cc:1199-1340) on GPUBatchArray1D.
class CublasLinearOpF : public ActOp {
public:
  typedef GPUArray4D<float> Kernel;
  typedef GPUArray1D<float> Bias;
  static shared_ptr<CublasLinearOpF> Make(size_t filters, ActVar x, shared_ptr<Var<Kernel>> kernel, shared_ptr<Var<Bias>> bias,
                                          shared_ptr<Context> ctx);
  CublasLinearOpF(size_t filters, ActVar x, shared_ptr<Var<Kernel>> kernel, shared_ptr<Var<Bias>> bias, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  string _debug_op_label() override { return "CublasLinearOp"; }
private:
  ActVar x_;
  shared_ptr<Var<Kernel>> kernel_;
  shared_ptr<Var<Bias>> bias_;
  size_t in_, out_;
};

// Bilinear x`scale` upsample of an H-strip (half-pixel centres, edges clamped).  The input is the strip
// halo-padded by one row and exchanged, so that each strip produces exactly its rows of the
// unpartitioned result; the gradient leaves the neighbours' shares in the halo rows, where the halo
// exchange's backward pass sums them.  Not in the reference: the segmentation head it never wrote.
class UpsampleBilinear2DOpF : public ActOp {
public:
  static vector<ActVar> MakeParallel(size_t scale, vector<ActVar> inputs, shared_ptr<Context> ctx);
  UpsampleBilinear2DOpF(size_t scale, size_t num_ranks, ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
private:
  ad_tensor4 low_view(Act& a) const;
  ActVar x_;
  size_t scale_, num_ranks_;
};

// Per-pixel softmax + negative log likelihood over the channel axis: the 3-D case of
// CudnnSoftmaxNLLLossOp that the reference asserts as unimplemented (src/op.cc:4190-4236).  A sink:
// forward fills loss[n][y][x] = logsumexp_c(x) - x[label], backward writes
// dx (+)= dloss * (softmax - onehot) with the per-pixel weight set by set_loss_weight (1 / pixels of
// the whole batch for a mean loss).  Labels are uint32 [N][h][W] of this rank's strip.
class CudnnSoftmaxNLLLoss2DOpF : public virtual Op {
public:
  static vector<shared_ptr<CudnnSoftmaxNLLLoss2DOpF>> MakeParallel(vector<ActVar> logits, shared_ptr<Context> ctx);
  CudnnSoftmaxNLLLoss2DOpF(ActVar x, shared_ptr<Context> ctx);
  void _forward(TxnId txn) override;
  void _backward(TxnId txn) override;
  void _set_grad_sink(TxnId) override {}
  string _debug_op_label() override { return "CudnnSoftmaxNLLLossOp"; }
  size_t rank() const { return x_->rank(); }
  size_t pixels() const { return n_ * hw_; }
  // Labels and per-pixel losses as graph variables, so that load_val / store_val reach them the way the reference's
  // tools do (net.labels with a Slice<uint32_t> reader, net.losses with a Slice<float> writer,
  // tools/train_imagenet.cc:220-243).  With `replica` set this operator is a copy of another rank's (every rank scores
  // the whole batch): it loads the same labels but does not advance the flat offset, and stores nothing.
  VarId label_var() const { return label_var_; }
  VarId loss_var() const { return loss_var_; }
  void set_replica(bool r) { replica_ = r; }
  size_t _load_val(TxnId txn, VarIdSet& vars, size_t offset, any* reader) override;
  size_t _store_val(TxnId txn, VarIdSet& vars, size_t offset, any* writer) override;
  void load_labels(const uint32_t* host);      // synchronous host -> device copy
  void set_loss_weight(float w);
  double loss_sum();                           // synchronous: sum of the per-pixel losses of the last forward (summed on the device, 8 bytes read back)
  void store_loss(float* host);                // synchronous: the per-pixel losses
private:
  ActVar x_;
  shared_ptr<Context> ctx_;
  size_t n_, hw_, classes_;
  uint32_t* labels_ = nullptr;
  float *loss_ = nullptr, *dloss_ = nullptr, *loss_sum_dev_ = nullptr;
  VarId label_var_, loss_var_;
  bool replica_ = false;
};

// Joins the per-rank sub-graphs under one root so that a single walk orders every rank's operators
// (the reference's graphs end in one scalar loss; a feature extractor has one output per rank).
class GroupSinkOp : public virtual Op {
public:
  explicit GroupSinkOp(vector<shared_ptr<Op>> members) { for (auto& m : members) inputs_.push_back(m); }
  void _forward(TxnId) override {}
  void _backward(TxnId) override {}
  void _set_grad_sink(TxnId) override {}
};

// Names of the reference's class templates.
template <typename V> using SpatialScatter2DOp = SpatialScatter2DOpF;
template <typename V> using SpatialGather2DOp = SpatialGather2DOpF;
template <typename V> using HaloPad2DOp = HaloPad2DOpF;
template <typename V> using HaloUnpad2DOp = HaloUnpad2DOpF;
template <typename V> using HaloRepad2DOp = HaloRepad2DOpF;
template <typename V> using HaloExch2DOp = HaloExch2DOpF;
template <typename V, typename K = GPUArray4D<float>, typename B = GPUArray1D<float>> using CudnnConv2DOp = CudnnConv2DOpF;
template <typename V> using CudnnPool2DOp = CudnnPool2DOpF;
template <typename S, typename V = Act, typename A = GPUArray1D<float>> using CudnnBatchNorm2DOp = CudnnBatchNorm2DOpF;
template <typename V> using CudnnActivationOp = CudnnActivationOpF;
template <typename V, typename J = SumJoin> using JoinOp = SumJoinOpF;
template <typename V> using UpsampleBilinear2DOp = UpsampleBilinear2DOpF;
template <typename V> using SpatialAllGather2DOp = SpatialAllGather2DOpF;
template <typename V> using BroadcastOp = BroadcastOpF;
template <typename V> using AllreduceOp = AllreduceOpF;
template <typename V> using ReduceOp = ReduceOpF;
template <typename V, typename K = GPUArray4D<float>, typename B = GPUArray1D<float>> using CublasLinearOp = CublasLinearOpF;
template <typename V> using CudnnSoftmaxNLLLossOp = CudnnSoftmaxNLLLoss2DOpF;

}  // namespace arraydiff
#endif
