// Operator bodies of the spatially parallel convolution path.  Every body is a sequence of
// calls into the arraydiff_b200 C ABI on the rank's stream; nothing here synchronises a device.
#include <cmath>
#include <cstdio>
#include <cstdlib>

#include "arraydiff/op.hh"

namespace arraydiff {

// ------------------------------------------------------------------ helpers
static GPUContext* gpu_of(const shared_ptr<Context>& ctx, size_t rank) {
  if (auto m = dynamic_cast<MultiGPUContext*>(ctx.get())) return m->device_context(rank).get();
  auto g = dynamic_cast<GPUContext*>(ctx.get());
  assert(g);
  return g;
}
// In a one-process-per-GPU run the per-rank lists hold only the local rank, so the grid size comes
// from the context, not from the list length.
static size_t num_ranks_of(const shared_ptr<Context>& ctx, size_t fallback) {
  if (auto m = dynamic_cast<MultiGPUContext*>(ctx.get())) return m->num_ranks();
  return fallback;
}
// the host float range behind a reader / writer: float* or Slice<float>
static float* host_floats(any* a) {
  if (auto hp = std::any_cast<float*>(a)) return *hp;
  if (auto sp = std::any_cast<Slice<float>>(a)) return sp->ptr;
  return nullptr;
}
GPUContext* ActOp::gpu() { return gpu_of(ctx_, rank_); }
MultiGPUContext* ActOp::mgpu() { return dynamic_cast<MultiGPUContext*>(ctx_.get()); }

void ActOp::alloc_output(Shape3D dim, size_t pad_w, size_t pad_h, size_t batch) {
  dim_ = dim;
  batch_ = batch;
  GPUContext* g = gpu();
  Shape3D off(pad_w, pad_h, 0);
  Shape3D padded(dim.shape[0] + 2 * pad_w, dim.shape[1] + 2 * pad_h, dim.shape[2]);
  Shape3D stride = padded.packed_stride();
  y_ = VarData<Act>([=]() { return Act::ZerosPadded(dim, off, stride, batch, g); });
}

size_t ActOp::_load_grad(TxnId txn, VarIdSet& vars, size_t offset, any* reader) {
  if (!vars.mask(y_.grad.var())) return offset;
  y_.grad.stamp(txn);
  Act& a = y_.grad.raw();
  if (reader) { float* hp = host_floats(reader); assert(hp); a.load_host_nchw(hp + offset, gpu()); }
  return offset + a.dim().flat_size() * a.batch_size();
}
size_t ActOp::_store_val(TxnId, VarIdSet& vars, size_t offset, any* writer) {
  if (!vars.mask(y_.val.var())) return offset;
  Act& a = y_.val.raw();
  if (writer) { float* hp = host_floats(writer); assert(hp); a.store_host_nchw(hp + offset, gpu()); }
  return offset + a.dim().flat_size() * a.batch_size();
}
size_t ActOp::_store_grad(TxnId, VarIdSet& vars, size_t offset, any* writer) {
  if (!vars.mask(y_.grad.var())) return offset;
  Act& a = y_.grad.raw();
  if (writer) { float* hp = host_floats(writer); assert(hp); a.store_host_nchw(hp + offset, gpu()); }
  return offset + a.dim().flat_size() * a.batch_size();
}

// Copies (or adds) a w x h window between two activations of equal channel count and storage.
// Coordinates are relative to each array's PADDED origin.  NCHW fp32 goes through the slice kernel
// as is; NHWC bf16 is the same kernel seen as one plane per image with rows of W*C elements.
static void copy_window(const Act& src, size_t sx, size_t sy, const Act& dst, size_t dx, size_t dy, size_t w, size_t h,
                        bool add, cudaStream_t s, const void* src_base = nullptr) {
  assert(src.storage() == dst.storage());
  if (!src_base) src_base = src.base_dptr();   // else: the same geometry at another address (a peer's copy)
  const Shape3D sp = src.padded_dim(), dp = dst.padded_dim();
  const uint32_t C = (uint32_t)sp.shape[2], N = (uint32_t)src.batch_size();
  assert(dp.shape[2] == C && dst.batch_size() == N);
  auto fn = add ? ad_slice2d_add_hw_nchw_packed : ad_slice2d_copy_hw_nchw_packed;
  if (src.storage() == COMPUTE_F32_NCHW) {
    AD_CHECK(fn(AD_F32, (uint32_t)w, (uint32_t)h, (uint32_t)sp.shape[0], (uint32_t)sp.shape[1], (uint32_t)dp.shape[0],
                (uint32_t)dp.shape[1], C, N, src_base, (uint32_t)sx, (uint32_t)sy, dst.base_dptr(), (uint32_t)dx,
                (uint32_t)dy, s));
  } else {
    AD_CHECK(fn(AD_BF16, (uint32_t)(w * C), (uint32_t)h, (uint32_t)(sp.shape[0] * C), (uint32_t)sp.shape[1],
                (uint32_t)(dp.shape[0] * C), (uint32_t)dp.shape[1], 1, N, src_base, (uint32_t)(sx * C), (uint32_t)sy,
                dst.base_dptr(), (uint32_t)(dx * C), (uint32_t)dy, s));
  }
}

// a writer of the interior covers the whole buffer exactly when there is no padding
static bool unpadded(Act& a) { return a.offset().shape[0] == 0 && a.offset().shape[1] == 0; }
static bool always(Act&) { return true; }

static function<void(Act*)> zero_init(GPUContext* g) {
  return [g](Act* a) { GPUConn c = g->conn(); a->zero(c); };
}

Shape3D Conv2DShape::calculate_output_shape(Shape3D in) const {
  // index 0 of each pair is the w axis, index 1 the h axis (reference src/op.cc:1356-1371)
  const size_t pw = halo_padded_input ? 0 : pad[0], ph = halo_padded_input ? 0 : pad[1];
  const size_t iw = in.shape[0] + (halo_padded_input ? 2 * pad[0] : 0), ih = in.shape[1] + (halo_padded_input ? 2 * pad[1] : 0);
  const size_t ow = (iw + 2 * pw - dilate[0] * (kernel[0] - 1) - 1) / stride[0] + 1;
  const size_t oh = (ih + 2 * ph - dilate[1] * (kernel[1] - 1) - 1) / stride[1] + 1;
  return Shape3D(ow, oh, filters);
}
Shape3D Pool2DShape::calculate_output_shape(Shape3D in) const {
  const size_t iw = in.shape[0] + (halo_padded_input ? 2 * pad[0] : 0), ih = in.shape[1] + (halo_padded_input ? 2 * pad[1] : 0);
  assert(halo_padded_input || (pad[0] == 0 && pad[1] == 0));
  return Shape3D((iw - window[0]) / stride[0] + 1, (ih - window[1]) / stride[1] + 1, in.shape[2]);
}

// ------------------------------------------------------------------ IOOp
template <> struct IOTraits<GPUArray1D<float>> {
  typedef GPUArray1D<float> A;
  static A alloc(Shape1D d, size_t, GPUContext* g) { return A(d, g); }
  static size_t size(A& a) { return a.flat_size(); }
  static float* dptr(A& a) { return a.dptr(); }
};
template <> struct IOTraits<GPUArray4D<float>> {
  typedef GPUArray4D<float> A;
  static A alloc(Shape4D d, size_t, GPUContext* g) { return A(d, g); }
  static size_t size(A& a) { return a.flat_size(); }
  static float* dptr(A& a) { return a.dptr(); }
};
template <> struct IOTraits<Act> {
  static Act alloc(Shape3D d, size_t batch, GPUContext* g) { return Act::Zeros(d, batch, g); }
  static size_t size(Act& a) { return a.dim().flat_size() * a.batch_size(); }
  static float* dptr(Act&) { return nullptr; }
};

static thread_local vector<string> g_scopes;
NameScope::NameScope(const string& name) { g_scopes.push_back(name); }
NameScope::~NameScope() { g_scopes.pop_back(); }
string NameScope::current() {
  string s;
  for (auto& p : g_scopes) { if (!s.empty()) s += "."; s += p; }
  return s;
}

template <typename A>
IOOp<A>::IOOp(typename A::Shape dim, size_t batch, InitFn init, size_t rank, shared_ptr<Context> ctx)
    : name_(NameScope::current()), dim_(dim), batch_(batch), rank_(rank), init_(init), ctx_(ctx) {
  GPUContext* g = gpu_of(ctx, rank);
  data_ = VarData<A>([=]() { return IOTraits<A>::alloc(dim, batch, g); });
}
template <typename A>
void IOOp<A>::_init(TxnId txn, std::mt19937_64* rng) {
  if (!init_) return;
  data_.val.stamp(txn);
  GPUConn conn = gpu_of(ctx_, rank_)->conn();   // the initialiser copies with this rank's device current
  init_(&data_.val.raw(), rng, ctx_);
}

// host <-> device movement of one IO variable; `flat` is float* (host) or GPUMemory<float> (device)
template <typename A>
static void io_move(A& a, any* flat, size_t offset, bool to_device, GPUContext* g) {
  const size_t n = IOTraits<A>::size(a);
  GPUConn conn = g->conn();
  if constexpr (std::is_same<A, Act>::value) {
    if (auto hr = std::any_cast<HostRows>(flat)) {
      assert(to_device);
      a.load_host_nchw_rows(hr->base, hr->full_h, hr->row0, g);
      return;
    }
  }
  if (float* hbase = host_floats(flat)) {
    float* host = hbase + offset;
    if constexpr (std::is_same<A, Act>::value) {
      if (to_device) a.load_host_nchw(host, g); else a.store_host_nchw(host, g);
    } else {
      float* d = IOTraits<A>::dptr(a);
      if (to_device) CUDA_CHECK(cudaMemcpyAsync(d, host, n * 4, cudaMemcpyHostToDevice, conn.stream()));
      else CUDA_CHECK(cudaMemcpyAsync(host, d, n * 4, cudaMemcpyDeviceToHost, conn.stream()));
      conn.sync();
    }
  } else if (auto dp = std::any_cast<GPUMemory<float>>(flat)) {
    if constexpr (std::is_same<A, Act>::value) {
      assert(0 && "activations move through host buffers");
    } else {
      float* d = IOTraits<A>::dptr(a);
      float* f = dp->dptr() + offset;
      if (to_device) CUDA_CHECK(cudaMemcpyAsync(d, f, n * 4, cudaMemcpyDeviceToDevice, conn.stream()));
      else CUDA_CHECK(cudaMemcpyAsync(f, d, n * 4, cudaMemcpyDeviceToDevice, conn.stream()));
    }
  } else {
    assert(0 && "reader/writer must hold float* or GPUMemory<float>");
  }
}
template <typename A>
size_t IOOp<A>::_load_val(TxnId txn, VarIdSet& vars, size_t offset, any* reader) {
  if (!vars.mask(data_.val.var())) return offset;
  data_.val.stamp(txn);
  A& a = data_.val.raw();
  if constexpr (std::is_same<A, Act>::value) {
    if (reader && full_h_ && !std::any_cast<HostRows>(reader)) {
      // the reader holds the whole batch: take this rank's rows of it (see set_rows_of_full)
      float* base = host_floats(reader);
      assert(base && "an activation input reads float* or Slice<float>");
      GPUContext* g = gpu_of(ctx_, rank_);
      if (host_nhwc_) a.load_host_nhwc_rows(base, full_h_, row0_, host_scale_, g);
      else a.load_host_nchw_rows(base, full_h_, row0_, g);
      return offset + IOTraits<A>::size(a);
    }
  }
  if (reader) io_move(a, reader, offset, true, gpu_of(ctx_, rank_));
  return offset + IOTraits<A>::size(a);
}
template <typename A>
size_t IOOp<A>::_load_grad(TxnId txn, VarIdSet& vars, size_t offset, any* reader) {
  if (!vars.mask(data_.grad.var())) return offset;
  data_.grad.stamp(txn);
  A& a = data_.grad.raw();
  if (reader) io_move(a, reader, offset, true, gpu_of(ctx_, rank_));
  return offset + IOTraits<A>::size(a);
}
template <typename A>
size_t IOOp<A>::_store_val(TxnId, VarIdSet& vars, size_t offset, any* writer) {
  if (!vars.mask(data_.val.var())) return offset;
  A& a = data_.val.raw();
  if (writer) {
    if (auto mp = std::any_cast<ParamManifest*>(writer)) {
      (*mp)->push_back(ParamManifestEntry{name_, offset, IOTraits<A>::size(a)});
      return offset + IOTraits<A>::size(a);
    }
  }
  if (writer) io_move(a, writer, offset, false, gpu_of(ctx_, rank_));
  return offset + IOTraits<A>::size(a);
}
template <typename A>
size_t IOOp<A>::_store_grad(TxnId, VarIdSet& vars, size_t offset, any* writer) {
  if (!vars.mask(data_.grad.var())) return offset;
  A& a = data_.grad.raw();
  if (writer) io_move(a, writer, offset, false, gpu_of(ctx_, rank_));
  return offset + IOTraits<A>::size(a);
}
template class IOOp<GPUArray1D<float>>;
template class IOOp<GPUArray4D<float>>;
template class IOOp<Act>;

// ------------------------------------------------------------------ scatter / gather
vector<ActVar> SpatialScatter2DOpF::MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (size_t r = 0; r < inputs.size(); ++r) out.push_back(make_shared<SpatialScatter2DOpF>(inputs[r]->rank(), num_ranks_of(ctx, inputs.size()), inputs[r], ctx));
  return out;
}
SpatialScatter2DOpF::SpatialScatter2DOpF(size_t rank, size_t num_ranks, ActVar x, shared_ptr<Context> ctx)
    : ActOp(rank, ctx), x_(x), num_ranks_(num_ranks) {
  inputs_.push_back(x);
  Shape3D d = x->shape();
  assert(d.shape[1] % num_ranks == 0);   // reference src/op.cc:2385-2387
  alloc_output(Shape3D(d.shape[0], d.shape[1] / num_ranks, d.shape[2]), 0, 0, x->batch_shape());
}
void SpatialScatter2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& y = y_.val.get_excl(txn, id());
  const size_t h = dim_.shape[1];
  copy_window(x, x.offset().shape[0], x.offset().shape[1] + rank_ * h, y, 0, 0, dim_.shape[0], h, false, conn.stream());
}
void SpatialScatter2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  if (!xd.grad.accumulate(txn, id(), zero_init(gpu()))) return;
  GPUConn conn = gpu()->conn();
  Act& dx = xd.grad.get_mut(txn, id());
  Act& dy = y_.grad.get(txn, id());
  const size_t h = dim_.shape[1];
  copy_window(dy, 0, 0, dx, dx.offset().shape[0], dx.offset().shape[1] + rank_ * h, dim_.shape[0], h, true, conn.stream());
}

vector<ActVar> SpatialGather2DOpF::MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (size_t r = 0; r < inputs.size(); ++r) out.push_back(make_shared<SpatialGather2DOpF>(inputs[r]->rank(), num_ranks_of(ctx, inputs.size()), inputs[r], ctx));
  return out;
}
SpatialGather2DOpF::SpatialGather2DOpF(size_t rank, size_t num_ranks, ActVar x, shared_ptr<Context> ctx)
    : ActOp(rank, ctx), x_(x), num_ranks_(num_ranks) {
  inputs_.push_back(x);
  Shape3D d = x->shape();
  alloc_output(Shape3D(d.shape[0], d.shape[1] * num_ranks, d.shape[2]), 0, 0, x->batch_shape());
}
void SpatialGather2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& y = y_.val.get_excl(txn, id());
  y.zero(conn);   // the other ranks' rows stay zero: summing the gathered tensors over ranks assembles the image
  const size_t h = x.dim().shape[1];
  copy_window(x, x.offset().shape[0], x.offset().shape[1], y, 0, rank_ * h, dim_.shape[0], h, false, conn.stream());
}
void SpatialGather2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(gpu()));
  if (!mode) return;
  GPUConn conn = gpu()->conn();
  Act& dx = xd.grad.get_mut(txn, id());
  Act& dy = y_.grad.get(txn, id());
  const size_t h = dx.dim().shape[1];
  copy_window(dy, 0, rank_ * h, dx, dx.offset().shape[0], dx.offset().shape[1], dim_.shape[0], h, mode == 1, conn.stream());
}

// ------------------------------------------------------------------ halo pad / unpad / repad
vector<ActVar> HaloPad2DOpF::MakeParallel(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (size_t r = 0; r < inputs.size(); ++r) out.push_back(make_shared<HaloPad2DOpF>(halo_pad, inputs[r]->rank(), inputs[r], ctx));
  return out;
}
HaloPad2DOpF::HaloPad2DOpF(size_t halo_pad, size_t rank, ActVar x, shared_ptr<Context> ctx) : ActOp(rank, ctx), x_(x), pad_(halo_pad) {
  inputs_.push_back(x);
  alloc_output(x->shape(), halo_pad, halo_pad, x->batch_shape());
}
void HaloPad2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& y = y_.val.get_excl(txn, id());
  // The pad cells were zeroed at allocation and nothing but the halo exchange ever writes them,
  // so only the interior moves (the reference re-zeroes on first use per transaction, src/op.cc:2580-2584).
  copy_window(x, x.offset().shape[0], x.offset().shape[1], y, pad_, pad_, dim_.shape[0], dim_.shape[1], false, conn.stream());
}
void HaloPad2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(gpu()));
  if (!mode) return;
  GPUConn conn = gpu()->conn();
  Act& dx = xd.grad.get_mut(txn, id());
  Act& dy = y_.grad.get(txn, id());
  copy_window(dy, pad_, pad_, dx, dx.offset().shape[0], dx.offset().shape[1], dim_.shape[0], dim_.shape[1], mode == 1, conn.stream());
}

vector<ActVar> HaloUnpad2DOpF::MakeParallel(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (size_t r = 0; r < inputs.size(); ++r) out.push_back(make_shared<HaloUnpad2DOpF>(halo_pad, inputs[r]->rank(), inputs[r], ctx));
  return out;
}
HaloUnpad2DOpF::HaloUnpad2DOpF(size_t halo_pad, size_t rank, ActVar x, shared_ptr<Context> ctx) : ActOp(rank, ctx), x_(x), pad_(halo_pad) {
  inputs_.push_back(x);
  alloc_output(x->shape(), 0, 0, x->batch_shape());
}
void HaloUnpad2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  assert(x.offset().shape[0] == pad_ && x.offset().shape[1] == pad_);
  copy_window(x, pad_, pad_, y_.val.get_excl(txn, id()), 0, 0, dim_.shape[0], dim_.shape[1], false, conn.stream());
}
void HaloUnpad2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  if (!xd.grad.accumulate(txn, id(), zero_init(gpu()))) return;
  GPUConn conn = gpu()->conn();
  copy_window(y_.grad.get(txn, id()), 0, 0, xd.grad.get_mut(txn, id()), pad_, pad_, dim_.shape[0], dim_.shape[1], true, conn.stream());
}

vector<ActVar> HaloRepad2DOpF::MakeParallel(size_t src_pad, size_t dst_pad, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (size_t r = 0; r < inputs.size(); ++r) out.push_back(make_shared<HaloRepad2DOpF>(src_pad, dst_pad, inputs[r]->rank(), inputs[r], ctx));
  return out;
}
HaloRepad2DOpF::HaloRepad2DOpF(size_t src_pad, size_t dst_pad, size_t rank, ActVar x, shared_ptr<Context> ctx)
    : ActOp(rank, ctx), x_(x), src_pad_(src_pad), dst_pad_(dst_pad) {
  inputs_.push_back(x);
  alloc_output(x->shape(), dst_pad, dst_pad, x->batch_shape());
}
void HaloRepad2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  copy_window(x_->data().val.get(txn, id()), src_pad_, src_pad_, y_.val.get_excl(txn, id()), dst_pad_, dst_pad_, dim_.shape[0],
              dim_.shape[1], false, conn.stream());
}
void HaloRepad2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  if (!xd.grad.accumulate(txn, id(), zero_init(gpu()))) return;
  GPUConn conn = gpu()->conn();
  copy_window(y_.grad.get(txn, id()), dst_pad_, dst_pad_, xd.grad.get_mut(txn, id()), src_pad_, src_pad_, dim_.shape[0],
              dim_.shape[1], true, conn.stream());
}

// ------------------------------------------------------------------ halo exchange (shared over ranks)
vector<ActVar> HaloExch2DOpF::MakeParallel(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  auto shared = make_shared<HaloExch2DOpF>(halo_pad, inputs, ctx);
  vector<ActVar> out;
  for (auto& x : inputs) out.push_back(make_shared<AliasOpF>(shared, x));
  return out;
}
HaloExch2DOpF::HaloExch2DOpF(size_t halo_pad, vector<ActVar> inputs, shared_ptr<Context> ctx) : pad_(halo_pad), xs_(inputs), ctx_(ctx) {
  for (auto& x : inputs) inputs_.push_back(x);
}
void HaloExch2DOpF::run(TxnId txn, bool reduce) {
  auto* m = dynamic_cast<MultiGPUContext*>(ctx_.get());
  assert(m);
  // All ranks record their block first, then every rank's kernel is launched: the reference's
  // group_start / halo_* / group_end sequence (src/op.cc:2977-3000) without its two device syncs.
  vector<size_t> local;
  for (size_t i = 0; i < xs_.size(); ++i) {
    const size_t r = xs_[i]->rank();
    if (!m->is_local(r)) continue;
    local.push_back(i);
    auto d = xs_[i]->data();
    GPUContext* g = m->device_context(r).get();
    Act* a;
    if (!reduce) {
      d.val.accumulate(txn, id(), nullptr);
      a = &d.val.get_mut(txn, id());
    } else {
      d.grad.accumulate(txn, id(), zero_init(g));
      a = &d.grad.get_mut(txn, id());
    }
    assert(a->offset().shape[0] == pad_ && a->offset().shape[1] == pad_);
    Spatial2DComm* comm = m->spatial_comm(r);
    const bool f32 = a->storage() == COMPUTE_F32_NCHW;
    comm->group_start();
    auto fn = reduce ? &Spatial2DComm::halo_reduce : &Spatial2DComm::halo_exchange;
    (comm->*fn)(a->base_dptr(), (uint32_t)pad_, (uint32_t)a->dim().shape[0], (uint32_t)a->dim().shape[1], (uint32_t)a->dim().shape[2],
                (uint32_t)a->batch_size(), f32 ? SPATIAL2D_TENSOR_NCHW : SPATIAL2D_TENSOR_NHWC,
                f32 ? SPATIAL2D_DATA_FLOAT : SPATIAL2D_DATA_BFLOAT16);
  }
  for (size_t i : local) {
    const size_t r = xs_[i]->rank();
    GPUConn conn = m->device_context(r)->conn();
    m->spatial_comm(r)->group_end(conn);
  }
}
void HaloExch2DOpF::_forward(TxnId txn) {
  if (done_fwd_ && *done_fwd_ == txn.raw_id()) return;
  done_fwd_ = txn.raw_id();
  run(txn, false);
}
void HaloExch2DOpF::_backward(TxnId txn) {
  if (done_bwd_ && *done_bwd_ == txn.raw_id()) return;
  done_bwd_ = txn.raw_id();
  run(txn, true);
}

// ------------------------------------------------------------------ convolution
shared_ptr<CudnnConv2DOpF> CudnnConv2DOpF::Make(Conv2DShape shape, ActVar x, shared_ptr<Var<Kernel>> kernel,
                                                shared_ptr<Var<Bias>> bias, shared_ptr<Context> ctx) {
  return make_shared<CudnnConv2DOpF>(shape, x, kernel, bias, ctx);
}
CudnnConv2DOpF::CudnnConv2DOpF(Conv2DShape shape, ActVar x, shared_ptr<Var<Kernel>> kernel, shared_ptr<Var<Bias>> bias,
                               shared_ptr<Context> ctx)
    : ActOp(x->rank(), ctx), shape_(shape), x_(x), kernel_(kernel), bias_(bias) {
  inputs_.push_back(x);
  inputs_.push_back(kernel);
  if (bias) inputs_.push_back(bias);
  in_dim_ = x->shape();
  alloc_output(shape.calculate_output_shape(in_dim_), 0, 0, x->batch_shape());
  if (gpu()->mode() == COMPUTE_BF16_NHWC) {
    const size_t C = in_dim_.shape[2], taps = shape.kernel[0] * shape.kernel[1];
    use_im2col_ = (C % 64) != 0;
    ck_ = use_im2col_ ? (taps * C + 63) / 64 * 64 : C;
    const size_t wcount = shape.filters * (use_im2col_ ? ck_ : taps * C);
    GPUContext* g = gpu();
    GPUConn conn = g->conn();
    w_bf16_ = g->arena().alloc(wcount * 2);
    dw_krsc_ = (float*)g->arena().alloc(wcount * 4);
    AD_CHECK(ad_fill_zero(w_bf16_, wcount * 2, conn.stream()));
    if (use_im2col_) {
      const size_t pix = dim_.shape[0] * dim_.shape[1] * batch_;
      im2col_ = g->arena().alloc(pix * ck_ * 2);
      AD_CHECK(ad_fill_zero(im2col_, pix * ck_ * 2, conn.stream()));
    }
  }
}

void CudnnConv2DOpF::fill_args(ad_conv2d_args& a, Act& x) {
  a = ad_conv2d_args();
  const bool f32 = x.storage() == COMPUTE_F32_NCHW;
  a.dtype = f32 ? AD_F32 : AD_BF16;
  a.layout = f32 ? AD_NCHW : AD_NHWC;
  const Shape3D pd = x.padded_dim();
  a.N = (uint32_t)x.batch_size();
  a.C = (uint32_t)pd.shape[2];
  a.K = (uint32_t)shape_.filters;
  a.kw = (uint32_t)shape_.kernel[0]; a.kh = (uint32_t)shape_.kernel[1];
  a.stride_w = (uint32_t)shape_.stride[0]; a.stride_h = (uint32_t)shape_.stride[1];
  a.dil_w = (uint32_t)shape_.dilate[0]; a.dil_h = (uint32_t)shape_.dilate[1];
  if (shape_.halo_padded_input) {
    // the kernel reads the padded buffer and is told pad 0 (reference src/op.cc:1354-1362, 1396-1410)
    assert(x.offset().shape[0] == shape_.pad[0] && x.offset().shape[1] == shape_.pad[1]);
    a.W = (uint32_t)pd.shape[0]; a.H = (uint32_t)pd.shape[1];
    a.x = x.base_dptr();
  } else {
    assert(x.offset().shape[0] == 0 && x.offset().shape[1] == 0 && "implicit padding needs a packed input");
    a.W = (uint32_t)x.dim().shape[0]; a.H = (uint32_t)x.dim().shape[1];
    a.pad_w = (uint32_t)shape_.pad[0]; a.pad_h = (uint32_t)shape_.pad[1];
    a.x = x.base_dptr();
  }
}

// bf16 KRSC copy of the fp32 KCRS master filter (columns padded to ck_ for the patch-matrix layer)
void CudnnConv2DOpF::refresh_filter(TxnId txn, cudaStream_t s) {
  Kernel& w = kernel_->data().val.get(txn, id());
  const long long K = (long long)shape_.filters, C = (long long)in_dim_.shape[2], kh = (long long)shape_.kernel[1], kw = (long long)shape_.kernel[0];
  ad_tensor4 src = {w.dptr(), AD_F32, (uint32_t)K, (uint32_t)C, (uint32_t)kh, (uint32_t)kw, C * kh * kw, kh * kw, kw, 1};
  const long long row = use_im2col_ ? (long long)ck_ : kh * kw * C;
  ad_tensor4 dst = {w_bf16_, AD_BF16, (uint32_t)K, (uint32_t)C, (uint32_t)kh, (uint32_t)kw, row, 1, kw * C, C};
  AD_CHECK(ad_convert(&src, &dst, 0, s));
}

void CudnnConv2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUContext* g = gpu();
  // Between processes the waits for the neighbours' halo rows of the exchange in front of this layer may still be
  // pending on the context: a stride-1 tensor-core layer convolves the output rows that need no halo first, then lets
  // the waits go, then adds the p rows at either edge -- the interior work overlaps the halo's flight, which the
  // reference forgoes by synchronising every device around each exchange (src/op.cc:2976, :3001).
  const size_t ph = shape_.pad[1], oh = dim_.shape[1];
  // The split costs two more launches (the boundary rows), ~25 us each on a persistent tensor-core kernel; the exchange
  // it hides is 15-25 us in flight.  It pays for layers of >= 150 GFLOP per strip (the 64-channel microbenchmark layer);
  // on the 1024 x 2048 segmentation net cut into 4 strips every layer is below that and the split step measured 3.5 %
  // slower.  ARRAYDIFF_B200_HALO_OVERLAP: "0" never splits, "2" always (the tests use it), anything else decides by size.
  const char* sw = getenv("ARRAYDIFF_B200_HALO_OVERLAP");
  const double gflop = 2e-9 * (double)batch_ * (double)shape_.filters * (double)in_dim_.shape[2] * (double)shape_.kernel[0] *
                       (double)shape_.kernel[1] * (double)dim_.shape[0] * (double)dim_.shape[1];
  const bool overlap = sw && sw[0] == '0' ? false : sw && sw[0] == '2' ? true : gflop >= 150.0;
  const bool split = overlap && g->has_pending() && g->mode() == COMPUTE_BF16_NHWC && shape_.halo_padded_input && !use_im2col_ &&
                     shape_.stride[0] == 1 && shape_.stride[1] == 1 && ph > 0 && oh > 2 * ph;
  GPUConn conn = split ? g->conn_deferred() : g->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& y = y_.val.get_excl(txn, id());
  ad_conv2d_args a;
  fill_args(a, x);
  a.bias = bias_ ? bias_->data().val.get(txn, id()).dptr() : nullptr;
  a.y = y.base_dptr();
  if (x.storage() == COMPUTE_F32_NCHW) {
    a.w = kernel_->data().val.get(txn, id()).dptr();
    AD_CHECK(ad_conv2d_fprop(&a, conn.stream()));
    return;
  }
  refresh_filter(txn, conn.stream());
  a.w = w_bf16_;
  if (use_im2col_) {
    ad_tensor4 xv = shape_.halo_padded_input ? x.view_base() : x.view_interior();
    assert(shape_.halo_padded_input || (shape_.pad[0] == 0 && shape_.pad[1] == 0));
    AD_CHECK(ad_im2col(&xv, a.kh, a.kw, a.stride_h, a.stride_w, a.dil_h, a.dil_w, (uint32_t)dim_.shape[1], (uint32_t)dim_.shape[0],
                       im2col_, (uint32_t)ck_, conn.stream()));
    a.x = im2col_; a.C = (uint32_t)ck_; a.H = (uint32_t)dim_.shape[1]; a.W = (uint32_t)dim_.shape[0];
    a.kh = a.kw = a.stride_h = a.stride_w = a.dil_h = a.dil_w = 1; a.pad_h = a.pad_w = 0;
  }
  g->reserve_scratch(16);
  a.scratch = g->status_word(); a.scratch_bytes = 16;
  if (split) {
    a.out_row_begin = (uint32_t)ph; a.out_row_count = (uint32_t)(oh - 2 * ph);
    AD_CHECK(ad_conv2d_fprop(&a, conn.stream()));
    g->finish_pending();
    a.out_row_begin = 0; a.out_row_count = (uint32_t)ph;
    AD_CHECK(ad_conv2d_fprop(&a, conn.stream()));
    a.out_row_begin = (uint32_t)(oh - ph);
    AD_CHECK(ad_conv2d_fprop(&a, conn.stream()));
    return;
  }
  AD_CHECK(ad_conv2d_fprop(&a, conn.stream()));
}

void CudnnConv2DOpF::_backward(TxnId txn) {
  GPUContext* g = gpu();
  GPUConn conn = g->conn();
  cudaStream_t s = conn.stream();
  Act& x = x_->data().val.get(txn, id());
  Act& dy = y_.grad.get(txn, id());
  ad_conv2d_args a;
  fill_args(a, x);
  a.y = dy.base_dptr();
  const bool f32 = x.storage() == COMPUTE_F32_NCHW;
  auto kd = kernel_->data();
  // filter (and bias) gradient: += after a once-per-transaction zero fill (reference src/op.cc:1651-1683)
  if (kd.grad.accumulate(txn, id(), [g](Kernel* k) { GPUConn c = g->conn(); AD_CHECK(ad_fill_zero(k->dptr(), k->flat_size() * 4, c.stream())); })) {
    Kernel& dw = kd.grad.get_mut(txn, id());
    float* db = nullptr;
    if (bias_) {
      auto bd = bias_->data();
      bd.grad.accumulate(txn, id(), [g](Bias* b) { GPUConn c = g->conn(); AD_CHECK(ad_fill_zero(b->dptr(), b->flat_size() * 4, c.stream())); });
      db = bd.grad.get_mut(txn, id()).dptr();
    }
    if (f32) {
      a.dw = dw.dptr(); a.db = db; a.accumulate = 1;
      AD_CHECK(ad_conv2d_wgrad(&a, s));
    } else {
      ad_conv2d_args b = a;
      if (use_im2col_) {
        b.x = im2col_; b.C = (uint32_t)ck_; b.H = (uint32_t)dim_.shape[1]; b.W = (uint32_t)dim_.shape[0];
        b.kh = b.kw = b.stride_h = b.stride_w = b.dil_h = b.dil_w = 1; b.pad_h = b.pad_w = 0;
      }
      const size_t need = ad_conv2d_scratch_bytes(&b, 2);
      if (!use_im2col_) {
        // Nothing reads a filter gradient before the end of the backward walk: it runs on the context's side stream
        // (with its own scratch), underneath the data gradient and the memory-bound operators of the layers below.
        // The fixed-order reduction of the partials adds straight into the (zero-initialised) KCRS variables.
        const char* sw = getenv("ARRAYDIFF_B200_WGRAD_OVERLAP");   // "0": keep the filter gradients on the main stream
        const bool overlap = !(sw && sw[0] == '0');
        cudaStream_t ws = s;
        if (overlap) {
          g->reserve_side_scratch(need);
          b.scratch = g->side_scratch(); b.scratch_bytes = g->side_scratch_size();
          ws = g->fork_side();
        } else {
          g->reserve_scratch(need);
          b.scratch = g->get_scratch(); b.scratch_bytes = g->scratch_size();
        }
        AD_CHECK(ad_fill_zero(b.scratch, 16, ws));
        b.dw = dw.dptr(); b.db = db; b.accumulate = 1; b.dw_kcrs = 1;
        AD_CHECK(ad_conv2d_wgrad(&b, ws));
      } else {
      g->reserve_scratch(need);
      b.scratch = g->get_scratch(); b.scratch_bytes = g->scratch_size();
      AD_CHECK(ad_fill_zero(b.scratch, 16, s));
      // patch-matrix layer: the filter gradient is produced with padded rows and then added into the KCRS
      // variable; the bias gradient is written straight into its variable (this op is the bias's only
      // consumer, so = equals +=)
      b.dw = dw_krsc_; b.db = db; b.accumulate = 0;
      AD_CHECK(ad_conv2d_wgrad(&b, s));
      const long long K = (long long)shape_.filters, C = (long long)in_dim_.shape[2], kh = (long long)shape_.kernel[1], kw = (long long)shape_.kernel[0];
      const long long row = use_im2col_ ? (long long)ck_ : kh * kw * C;
      ad_tensor4 src = {dw_krsc_, AD_F32, (uint32_t)K, (uint32_t)C, (uint32_t)kh, (uint32_t)kw, row, 1, kw * C, C};
      ad_tensor4 dst = {dw.dptr(), AD_F32, (uint32_t)K, (uint32_t)C, (uint32_t)kh, (uint32_t)kw, C * kh * kw, kh * kw, kw, 1};
      AD_CHECK(ad_convert(&src, &dst, 1, s));
      }
    }
  }
  // data gradient over the whole padded extent, halo rows included (reference src/op.cc:1687-1724)
  if (use_im2col_) return;   // first layer: its input is data and takes no gradient
  auto xd = x_->data();
  // halo-padded input: the gradient covers the whole padded extent; packed input: the whole packed extent
  if (const int mode = xd.grad.accumulate_full(txn, id(), shape_.halo_padded_input ? always : unpadded, zero_init(g))) {
    Act& dx = xd.grad.get_mut(txn, id());
    a.dx = dx.base_dptr();
    a.accumulate = mode == 1 ? 1 : 0;
    if (f32) {
      a.w = kd.val.get(txn, id()).dptr();
      AD_CHECK(ad_conv2d_dgrad(&a, s));
    } else {
      a.w = w_bf16_;
      if (shape_.halo_padded_input && dx.offset().shape[0] > 0) {
        // the W-pad columns of a gradient buffer are never read (pad / exchange backward take interior columns)
        a.dx_col_begin = (uint32_t)dx.offset().shape[0];
        a.dx_col_count = (uint32_t)dx.dim().shape[0];
      }
      const size_t need = ad_conv2d_scratch_bytes(&a, 1);
      g->reserve_scratch(need);
      a.scratch = g->get_scratch(); a.scratch_bytes = g->scratch_size();
      AD_CHECK(ad_fill_zero(a.scratch, 16, s));
      AD_CHECK(ad_conv2d_dgrad(&a, s));
    }
  }
}

// ------------------------------------------------------------------ pooling
shared_ptr<CudnnPool2DOpF> CudnnPool2DOpF::Make(Pool2DShape shape, ActVar x, shared_ptr<Context> ctx) {
  return make_shared<CudnnPool2DOpF>(shape, x, ctx);
}
vector<ActVar> CudnnPool2DOpF::MakeParallel(Pool2DShape shape, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (auto& x : inputs) out.push_back(Make(shape, x, ctx));
  return out;
}
CudnnPool2DOpF::CudnnPool2DOpF(Pool2DShape shape, ActVar x, shared_ptr<Context> ctx) : ActOp(x->rank(), ctx), shape_(shape), x_(x) {
  inputs_.push_back(x);
  assert((shape.pooling == kMaxPool || !shape.halo_padded_input) && "average pooling takes an unpadded input");
  alloc_output(shape.calculate_output_shape(x->shape()), 0, 0, x->batch_shape());
}
void CudnnPool2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  if (shape_.halo_padded_input) assert(x.offset().shape[0] == shape_.pad[0] && x.offset().shape[1] == shape_.pad[1]);   // reference src/op.cc:3427-3428
  ad_tensor4 xv = shape_.halo_padded_input ? x.view_base() : x.view_interior();
  ad_tensor4 yv = y_.val.get_excl(txn, id()).view_interior();
  if (shape_.pooling == kAveragePool) {
    AD_CHECK(ad_avgpool2d_fwd(&xv, &yv, (uint32_t)shape_.window[1], (uint32_t)shape_.window[0], (uint32_t)shape_.stride[1],
                              (uint32_t)shape_.stride[0], conn.stream()));
    return;
  }
  AD_CHECK(ad_maxpool2d_fwd(&xv, &yv, (uint32_t)shape_.window[1], (uint32_t)shape_.window[0], (uint32_t)shape_.stride[1],
                            (uint32_t)shape_.stride[0], conn.stream()));
}
void CudnnPool2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), shape_.halo_padded_input ? always : unpadded, zero_init(gpu()));
  if (!mode) return;
  GPUConn conn = gpu()->conn();
  Act& x = xd.val.get(txn, id());
  Act& dx = xd.grad.get_mut(txn, id());
  ad_tensor4 xv = shape_.halo_padded_input ? x.view_base() : x.view_interior();
  ad_tensor4 dxv = shape_.halo_padded_input ? dx.view_base() : dx.view_interior();
  ad_tensor4 dyv = y_.grad.get(txn, id()).view_interior();
  if (shape_.pooling == kAveragePool) {
    AD_CHECK(ad_avgpool2d_bwd(&dyv, &dxv, (uint32_t)shape_.window[1], (uint32_t)shape_.window[0], (uint32_t)shape_.stride[1],
                              (uint32_t)shape_.stride[0], mode == 1 ? 1 : 0, conn.stream()));
    return;
  }
  AD_CHECK(ad_maxpool2d_bwd(&xv, &dyv, &dxv, (uint32_t)shape_.window[1], (uint32_t)shape_.window[0], (uint32_t)shape_.stride[1],
                            (uint32_t)shape_.stride[0], mode == 1 ? 1 : 0, conn.stream()));
}

// ------------------------------------------------------------------ batch norm (+ fused ReLU)
static IOOp<GPUArray1D<float>>::InitFn const_init(float v) {
  return [v](GPUArray1D<float>* a, std::mt19937_64*, shared_ptr<Context>) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceSynchronize();   // the context streams do not synchronise with the default stream
    AD_CHECK(ad_array_set_constant(a->flat_size(), v, a->dptr(), nullptr));
    cudaDeviceSynchronize();
  };
}
CudnnBatchNorm2DOpF::Parts CudnnBatchNorm2DOpF::Make(size_t channels, shared_ptr<bool> switch_var, ActVar x, shared_ptr<Context> ctx) {
  Parts p;
  typedef IOOp<Stat> S;
  const size_t r = x->rank();
  p.scale = S::Make(Shape1D(channels), 1, const_init(1.f), r, ctx);
  p.shift = S::Make(Shape1D(channels), 1, const_init(0.f), r, ctx);
  p.scale->set_name(NameScope::current() + ".scale");
  p.shift->set_name(NameScope::current() + ".shift");
  p.batch_mean = S::Make(Shape1D(channels), 1, nullptr, r, ctx);
  p.batch_variance = S::Make(Shape1D(channels), 1, nullptr, r, ctx);
  p.fixed_mean = S::Make(Shape1D(channels), 1, const_init(0.f), r, ctx);
  p.fixed_variance = S::Make(Shape1D(channels), 1, const_init(1.f), r, ctx);
  p.op = make_shared<CudnnBatchNorm2DOpF>(switch_var, x, &p, ctx);
  return p;
}
CudnnBatchNorm2DOpF::CudnnBatchNorm2DOpF(shared_ptr<bool> switch_var, ActVar x, Parts* parts, shared_ptr<Context> ctx)
    : ActOp(x->rank(), ctx), switch_var_(switch_var), x_(x), scale_(parts->scale), shift_(parts->shift),
      batch_mean_(parts->batch_mean), batch_variance_(parts->batch_variance), fixed_mean_(parts->fixed_mean),
      fixed_variance_(parts->fixed_variance) {
  inputs_.push_back(x);
  inputs_.push_back(scale_);
  inputs_.push_back(shift_);
  // statistics are graph variables too: the optimizer reads the batch statistics and loads the running ones
  inputs_.push_back(batch_mean_);
  inputs_.push_back(batch_variance_);
  inputs_.push_back(fixed_mean_);
  inputs_.push_back(fixed_variance_);
  alloc_output(x->shape(), 0, 0, x->batch_shape());
  const size_t C = x->shape().shape[2];
  save_mean_ = (float*)gpu()->arena().alloc(C * 4);
  save_invstd_ = (float*)gpu()->arena().alloc(C * 4);
}
void CudnnBatchNorm2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUContext* g = gpu();
  GPUConn conn = g->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& y = y_.val.get_excl(txn, id());
  const uint32_t C = (uint32_t)dim_.shape[2];
  g->reserve_scratch(ad_bn_scratch_bytes(C));
  ad_tensor4 xv = x.view_interior(), yv = y.view_interior();
  if (switch_var_ && *switch_var_) {
    // validation: normalise with the running statistics (reference src/op.cc:3964-3978)
    AD_CHECK(ad_bn_fwd_inference(&xv, &yv, scale_->data().val.get(txn, id()).dptr(), shift_->data().val.get(txn, id()).dptr(),
                                 fixed_mean_->data().val.raw().dptr(), fixed_variance_->data().val.raw().dptr(), save_invstd_, 1.0e-5f,
                                 relu_ ? 1 : 0, conn.stream()));
    return;
  }
  batch_mean_->data().val.stamp(txn);
  batch_variance_->data().val.stamp(txn);
  AD_CHECK(ad_bn_fwd_train(&xv, &yv, scale_->data().val.get(txn, id()).dptr(), shift_->data().val.get(txn, id()).dptr(), save_mean_,
                           save_invstd_, batch_variance_->data().val.raw().dptr(), 1.0e-5f, relu_ ? 1 : 0, g->get_scratch(),
                           g->scratch_size(), conn.stream()));
  // batch_mean mirrors the saved mean (what the optimizer's running-average step consumes)
  CUDA_CHECK(cudaMemcpyAsync(batch_mean_->data().val.raw().dptr(), save_mean_, C * 4, cudaMemcpyDeviceToDevice, conn.stream()));
}
void CudnnBatchNorm2DOpF::_backward(TxnId txn) {
  assert(!(switch_var_ && *switch_var_) && "no backward pass with fixed statistics (reference src/op.cc:4078-4080)");
  GPUContext* g = gpu();
  auto xd = x_->data();
  auto zero1 = [g](Stat* a) { GPUConn c = g->conn(); AD_CHECK(ad_fill_zero(a->dptr(), a->flat_size() * 4, c.stream())); };
  auto sd = scale_->data(), hd = shift_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(g));
  if (!mode) return;
  sd.grad.accumulate(txn, id(), zero1);
  hd.grad.accumulate(txn, id(), zero1);
  GPUConn conn = g->conn();
  const uint32_t C = (uint32_t)dim_.shape[2];
  g->reserve_scratch(ad_bn_scratch_bytes(C));
  ad_tensor4 xv = xd.val.get(txn, id()).view_interior(), dyv = y_.grad.get(txn, id()).view_interior(),
             dxv = xd.grad.get_mut(txn, id()).view_interior();
  AD_CHECK(ad_bn_bwd(&xv, &dyv, &dxv, sd.val.get(txn, id()).dptr(), hd.val.get(txn, id()).dptr(), save_mean_, save_invstd_,
                     sd.grad.get_mut(txn, id()).dptr(), hd.grad.get_mut(txn, id()).dptr(), relu_ ? 1 : 0, mode == 1 ? 1 : 0, g->get_scratch(),
                     g->scratch_size(), conn.stream()));
}

// ------------------------------------------------------------------ ReLU, residual sum
ActVar CudnnActivationOpF::Make(ActivationKind, ActVar x, shared_ptr<Context> ctx) {
  return make_shared<CudnnActivationOpF>(x, ctx);
}
CudnnActivationOpF::CudnnActivationOpF(ActVar x, shared_ptr<Context> ctx) : ActOp(x->rank(), ctx), x_(x) {
  inputs_.push_back(x);
  alloc_output(x->shape(), 0, 0, x->batch_shape());
}
void CudnnActivationOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  ad_tensor4 xv = x_->data().val.get(txn, id()).view_interior(), yv = y_.val.get_excl(txn, id()).view_interior();
  AD_CHECK(ad_relu_fwd(&xv, &yv, conn.stream()));
}
void CudnnActivationOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(gpu()));
  if (!mode) return;
  GPUConn conn = gpu()->conn();
  ad_tensor4 xv = xd.val.get(txn, id()).view_interior(), dyv = y_.grad.get(txn, id()).view_interior(),
             dxv = xd.grad.get_mut(txn, id()).view_interior();
  AD_CHECK(ad_relu_bwd(&xv, &dyv, &dxv, mode == 1 ? 1 : 0, conn.stream()));
}

ActVar SumJoinOpF::Make(vector<ActVar> xs, shared_ptr<Context> ctx) { return make_shared<SumJoinOpF>(xs, ctx); }
SumJoinOpF::SumJoinOpF(vector<ActVar> xs, shared_ptr<Context> ctx) : ActOp(xs.at(0)->rank(), ctx), xs_(xs) {
  assert(xs.size() >= 2);
  for (auto& x : xs) { inputs_.push_back(x); assert(x->shape() == xs[0]->shape()); }
  alloc_output(xs[0]->shape(), 0, 0, xs[0]->batch_shape());
}
void SumJoinOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  ad_tensor4 yv = y_.val.get_excl(txn, id()).view_interior();
  ad_tensor4 a = xs_[0]->data().val.get(txn, id()).view_interior(), b = xs_[1]->data().val.get(txn, id()).view_interior();
  AD_CHECK(ad_add(&a, &b, &yv, conn.stream()));
  for (size_t i = 2; i < xs_.size(); ++i) {
    ad_tensor4 c = xs_[i]->data().val.get(txn, id()).view_interior();
    AD_CHECK(ad_add(&yv, &c, &yv, conn.stream()));
  }
}
void SumJoinOpF::_backward(TxnId txn) {
  GPUConn conn = gpu()->conn();
  ad_tensor4 dyv = y_.grad.get(txn, id()).view_interior();
  for (auto& x : xs_) {
    auto xd = x->data();
    const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(gpu()));
    if (!mode) continue;
    ad_tensor4 dxv = xd.grad.get_mut(txn, id()).view_interior();
    AD_CHECK(ad_convert(&dyv, &dxv, mode == 1 ? 1 : 0, conn.stream()));
  }
}

// ------------------------------------------------------------------ all-gather of strips / reduce-scatter of gradients
AllGatherOutF::AllGatherOutF(shared_ptr<SpatialAllGather2DOpF> shared, ActVar strip, size_t num_ranks, shared_ptr<Context> ctx)
    : ActOp(strip->rank(), ctx) {
  inputs_.push_back(shared);
  Shape3D d = strip->shape();
  alloc_output(Shape3D(d.shape[0], d.shape[1] * num_ranks, d.shape[2]), 0, 0, strip->batch_shape());
}
vector<ActVar> SpatialAllGather2DOpF::MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx) {
  auto shared = make_shared<SpatialAllGather2DOpF>(inputs, ctx);
  vector<ActVar> out;
  for (auto& x : inputs) {
    auto o = make_shared<AllGatherOutF>(shared, x, shared->num_ranks_, ctx);
    shared->outs_.push_back(o.get());
    out.push_back(o);
  }
  return out;
}
SpatialAllGather2DOpF::SpatialAllGather2DOpF(vector<ActVar> inputs, shared_ptr<Context> ctx)
    : xs_(inputs), ctx_(ctx), num_ranks_(num_ranks_of(ctx, inputs.size())) {
  for (auto& x : inputs) inputs_.push_back(x);
}
// Between processes: tell every peer that my strip (or my gradient) of this exchange may be read, then wait
// (bounded) for theirs.  Every rank calls the gathers in the same order, so the round number agrees.
void SpatialAllGather2DOpF::wait_peers(size_t rank, cudaStream_t s) {
  auto* m = dynamic_cast<MultiGPUContext*>(ctx_.get());
  Spatial2DComm* comm = m->spatial_comm(rank);
  const uint64_t k = comm->next_phase_epoch();
  GPUContext* g = m->device_context(rank).get();
  for (size_t q = 0; q < num_ranks_; ++q)
    if (q != rank) AD_CHECK(ad_flag_signal_rel((uint64_t*)m->peer_ptr(comm->gather_flags() + rank, rank, q), comm->epoch_base(), k, s));
  for (size_t q = 0; q < num_ranks_; ++q)
    if (q != rank) AD_CHECK(ad_flag_wait_rel(comm->gather_flags() + q, comm->epoch_base(), k, 2000000000ull, g->status_word(), s));
}
// stream `to` waits for everything issued so far on stream `from`
static void order_after(cudaStream_t to, cudaStream_t from) {
  cudaEvent_t e;
  CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  CUDA_CHECK(cudaEventRecord(e, from));
  CUDA_CHECK(cudaStreamWaitEvent(to, e, 0));
  CUDA_CHECK(cudaEventDestroy(e));
}
void SpatialAllGather2DOpF::_forward(TxnId txn) {
  if (done_fwd_ && *done_fwd_ == txn.raw_id()) return;
  done_fwd_ = txn.raw_id();
  auto* m = dynamic_cast<MultiGPUContext*>(ctx_.get());
  assert(m);
  for (size_t i = 0; i < xs_.size(); ++i) {
    const size_t r = xs_[i]->rank();
    if (!m->is_local(r)) continue;
    auto yd = outs_[i]->data();
    if (!yd.val.overwrite(txn, id())) continue;
    GPUContext* g = m->device_context(r).get();
    GPUConn conn = g->conn();
    Act& x = xs_[i]->data().val.get(txn, id());
    Act& y = yd.val.get_excl(txn, id());
    const size_t w = x.dim().shape[0], h = x.dim().shape[1], ox = x.offset().shape[0], oy = x.offset().shape[1];
    copy_window(x, ox, oy, y, 0, r * h, w, h, false, conn.stream());
    if (num_ranks_ == 1) continue;
    if (m->distributed()) {
      wait_peers(r, conn.stream());
      for (size_t q = 0; q < num_ranks_; ++q)
        if (q != r) copy_window(x, ox, oy, y, 0, q * h, w, h, false, conn.stream(), m->peer_ptr(x.base_dptr(), r, q));
      continue;
    }
    for (size_t j = 0; j < xs_.size(); ++j) {
      const size_t q = xs_[j]->rank();
      if (q == r) continue;
      // what has been issued on rank q's stream so far includes the producer of its strip
      order_after(conn.stream(), m->device_context(q)->stream());
      Act& xs = xs_[j]->data().val.get(txn, id());
      copy_window(xs, xs.offset().shape[0], xs.offset().shape[1], y, 0, q * h, w, h, false, conn.stream());
    }
  }
}
void SpatialAllGather2DOpF::_backward(TxnId txn) {
  if (done_bwd_ && *done_bwd_ == txn.raw_id()) return;
  done_bwd_ = txn.raw_id();
  auto* m = dynamic_cast<MultiGPUContext*>(ctx_.get());
  for (size_t i = 0; i < xs_.size(); ++i) {
    const size_t r = xs_[i]->rank();
    if (!m->is_local(r)) continue;
    GPUContext* g = m->device_context(r).get();
    auto xd = xs_[i]->data();
    const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(g));
    if (!mode) continue;
    GPUConn conn = g->conn();
    Act& dx = xd.grad.get_mut(txn, id());
    Act& dy = outs_[i]->data().grad.get(txn, id());
    const size_t w = dx.dim().shape[0], h = dx.dim().shape[1], ox = dx.offset().shape[0], oy = dx.offset().shape[1];
    // peers in rank order, the own share in its place: the sum does not depend on which rank computes it
    bool first = mode != 1;
    auto add_from = [&](const Act& src, const void* base) {
      copy_window(src, 0, r * h, dx, ox, oy, w, h, !first, conn.stream(), base);
      first = false;
    };
    if (num_ranks_ > 1 && m->distributed()) wait_peers(r, conn.stream());
    for (size_t q = 0; q < num_ranks_; ++q) {
      if (q == r) { add_from(dy, nullptr); continue; }
      if (m->distributed()) { add_from(dy, m->peer_ptr(dy.base_dptr(), r, q)); continue; }
      for (size_t j = 0; j < xs_.size(); ++j) {
        if (xs_[j]->rank() != q) continue;
        order_after(conn.stream(), m->device_context(q)->stream());
        add_from(outs_[j]->data().grad.get(txn, id()), nullptr);
      }
    }
  }
}

// ------------------------------------------------------------------ broadcast / allreduce / reduce (one process)
CollectiveOutF::CollectiveOutF(shared_ptr<Op> shared, ActVar like, size_t rank, shared_ptr<Context> ctx) : ActOp(rank, ctx) {
  inputs_.push_back(shared);
  alloc_output(like->shape(), 0, 0, like->batch_shape());
}
static MultiGPUContext* in_process(const shared_ptr<Context>& ctx) {
  auto* m = dynamic_cast<MultiGPUContext*>(ctx.get());
  assert(m && !m->distributed() && "graph collectives serve one-process contexts; between processes use scatter-on-load / SpatialAllGather2DOp");
  return m;
}
// dst (=|+=) src on dst's rank, after everything issued so far on src's rank
static void pull(MultiGPUContext* m, size_t dst_rank, Act& dst, size_t src_rank, Act& src, bool add) {
  GPUConn conn = m->device_context(dst_rank)->conn();
  if (src_rank != dst_rank) order_after(conn.stream(), m->device_context(src_rank)->stream());
  ad_tensor4 s = src.view_interior(), d = dst.view_interior();
  AD_CHECK(ad_convert(&s, &d, add ? 1 : 0, conn.stream()));
}

vector<ActVar> BroadcastOpF::MakeParallel(size_t root, ActVar x, shared_ptr<Context> ctx) {
  auto shared = make_shared<BroadcastOpF>(root, x, ctx);
  vector<ActVar> out;
  for (size_t r = 0; r < in_process(ctx)->num_ranks(); ++r) {
    auto o = make_shared<CollectiveOutF>(shared, x, r, ctx);
    shared->outs_.push_back(o.get());
    out.push_back(o);
  }
  return out;
}
BroadcastOpF::BroadcastOpF(size_t root, ActVar x, shared_ptr<Context> ctx) : root_(root), x_(x), ctx_(ctx) {
  assert(x->rank() == root);
  inputs_.push_back(x);
}
void BroadcastOpF::_forward(TxnId txn) {
  if (done_fwd_ && *done_fwd_ == txn.raw_id()) return;
  done_fwd_ = txn.raw_id();
  auto* m = in_process(ctx_);
  Act& x = x_->data().val.get(txn, id());
  for (size_t r = 0; r < outs_.size(); ++r) {
    auto yd = outs_[r]->data();
    if (!yd.val.overwrite(txn, id())) continue;
    pull(m, r, yd.val.get_excl(txn, id()), root_, x, false);
  }
}
void BroadcastOpF::_backward(TxnId txn) {
  if (done_bwd_ && *done_bwd_ == txn.raw_id()) return;
  done_bwd_ = txn.raw_id();
  auto* m = in_process(ctx_);
  auto xd = x_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(m->device_context(root_).get()));
  if (!mode) return;
  bool add = mode == 1;
  for (size_t r = 0; r < outs_.size(); ++r) {
    if (!outs_[r]->data().grad.written_in(txn)) continue;   // a rank whose copy nobody used
    pull(m, root_, xd.grad.get_mut(txn, id()), r, outs_[r]->data().grad.get(txn, id()), add);
    add = true;
  }
}

vector<ActVar> AllreduceOpF::MakeParallel(vector<ActVar> inputs, shared_ptr<Context> ctx) {
  auto shared = make_shared<AllreduceOpF>(inputs, ctx);
  vector<ActVar> out;
  for (auto& x : inputs) {
    auto o = make_shared<CollectiveOutF>(shared, x, x->rank(), ctx);
    shared->outs_.push_back(o.get());
    out.push_back(o);
  }
  return out;
}
AllreduceOpF::AllreduceOpF(vector<ActVar> inputs, shared_ptr<Context> ctx) : xs_(inputs), ctx_(ctx) {
  in_process(ctx);
  for (auto& x : inputs) inputs_.push_back(x);
}
void AllreduceOpF::_forward(TxnId txn) {
  if (done_fwd_ && *done_fwd_ == txn.raw_id()) return;
  done_fwd_ = txn.raw_id();
  auto* m = in_process(ctx_);
  for (size_t i = 0; i < xs_.size(); ++i) {
    auto yd = outs_[i]->data();
    if (!yd.val.overwrite(txn, id())) continue;
    for (size_t j = 0; j < xs_.size(); ++j)    // rank order: the same bits on every rank
      pull(m, xs_[i]->rank(), yd.val.get_excl(txn, id()), xs_[j]->rank(), xs_[j]->data().val.get(txn, id()), j != 0);
  }
}
void AllreduceOpF::_backward(TxnId txn) {
  if (done_bwd_ && *done_bwd_ == txn.raw_id()) return;
  done_bwd_ = txn.raw_id();
  auto* m = in_process(ctx_);
  for (size_t i = 0; i < xs_.size(); ++i) {
    auto xd = xs_[i]->data();
    const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(m->device_context(xs_[i]->rank()).get()));
    if (!mode) continue;
    bool add = mode == 1;
    for (size_t j = 0; j < xs_.size(); ++j) {
      if (!outs_[j]->data().grad.written_in(txn)) continue;
      pull(m, xs_[i]->rank(), xd.grad.get_mut(txn, id()), xs_[j]->rank(), outs_[j]->data().grad.get(txn, id()), add);
      add = true;
    }
  }
}

ActVar ReduceOpF::MakeParallel(size_t root, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  auto shared = make_shared<ReduceOpF>(root, inputs, ctx);
  auto o = make_shared<CollectiveOutF>(shared, inputs.at(0), root, ctx);
  shared->out_ = o.get();
  return o;
}
ReduceOpF::ReduceOpF(size_t root, vector<ActVar> inputs, shared_ptr<Context> ctx) : root_(root), xs_(inputs), ctx_(ctx) {
  in_process(ctx);
  for (auto& x : inputs) inputs_.push_back(x);
}
void ReduceOpF::_forward(TxnId txn) {
  if (done_fwd_ && *done_fwd_ == txn.raw_id()) return;
  done_fwd_ = txn.raw_id();
  auto* m = in_process(ctx_);
  auto yd = out_->data();
  if (!yd.val.overwrite(txn, id())) return;
  for (size_t j = 0; j < xs_.size(); ++j)
    pull(m, root_, yd.val.get_excl(txn, id()), xs_[j]->rank(), xs_[j]->data().val.get(txn, id()), j != 0);
}
void ReduceOpF::_backward(TxnId txn) {
  if (done_bwd_ && *done_bwd_ == txn.raw_id()) return;
  done_bwd_ = txn.raw_id();
  auto* m = in_process(ctx_);
  Act& dy = out_->data().grad.get(txn, id());
  for (auto& x : xs_) {
    auto xd = x->data();
    const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(m->device_context(x->rank()).get()));
    if (!mode) continue;
    pull(m, x->rank(), xd.grad.get_mut(txn, id()), root_, dy, mode == 1);
  }
}

// ------------------------------------------------------------------ fully connected
shared_ptr<CublasLinearOpF> CublasLinearOpF::Make(size_t filters, ActVar x, shared_ptr<Var<Kernel>> kernel, shared_ptr<Var<Bias>> bias,
                                                  shared_ptr<Context> ctx) {
  return make_shared<CublasLinearOpF>(filters, x, kernel, bias, ctx);
}
CublasLinearOpF::CublasLinearOpF(size_t filters, ActVar x, shared_ptr<Var<Kernel>> kernel, shared_ptr<Var<Bias>> bias, shared_ptr<Context> ctx)
    : ActOp(x->rank(), ctx), x_(x), kernel_(kernel), bias_(bias), out_(filters) {
  inputs_.push_back(x);
  inputs_.push_back(kernel);
  if (bias) inputs_.push_back(bias);
  Shape3D d = x->shape();
  assert(d.shape[0] == 1 && d.shape[1] == 1 && "the linear layer takes [batch][features] (flatten after a global pool)");
  in_ = d.shape[2];
  alloc_output(Shape3D(1, 1, filters), 0, 0, x->batch_shape());
}
void CublasLinearOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& y = y_.val.get_excl(txn, id());
  assert(x.offset().shape[0] == 0 && x.offset().shape[1] == 0);
  const int dt = x.storage() == COMPUTE_F32_NCHW ? AD_F32 : AD_BF16;
  AD_CHECK(ad_linear_fwd(dt, (uint32_t)x.batch_size(), (uint32_t)in_, (uint32_t)out_, x.base_dptr(),
                         kernel_->data().val.get(txn, id()).dptr(), bias_ ? bias_->data().val.get(txn, id()).dptr() : nullptr,
                         y.base_dptr(), conn.stream()));
}
void CublasLinearOpF::_backward(TxnId txn) {
  GPUContext* g = gpu();
  GPUConn conn = g->conn();
  Act& x = x_->data().val.get(txn, id());
  Act& dy = y_.grad.get(txn, id());
  const int dt = x.storage() == COMPUTE_F32_NCHW ? AD_F32 : AD_BF16;
  auto kd = kernel_->data();
  float* dw = nullptr;
  float* db = nullptr;
  auto zero_k = [g](Kernel* a) { GPUConn c = g->conn(); AD_CHECK(ad_fill_zero(a->dptr(), a->flat_size() * 4, c.stream())); };
  auto zero_b = [g](Bias* a) { GPUConn c = g->conn(); AD_CHECK(ad_fill_zero(a->dptr(), a->flat_size() * 4, c.stream())); };
  if (kd.grad.accumulate(txn, id(), zero_k)) dw = kd.grad.get_mut(txn, id()).dptr();
  if (bias_ && dw) { auto bd = bias_->data(); bd.grad.accumulate(txn, id(), zero_b); db = bd.grad.get_mut(txn, id()).dptr(); }
  auto xd = x_->data();
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(g));
  void* dxp = mode ? xd.grad.get_mut(txn, id()).base_dptr() : nullptr;
  if (!dw && !dxp) return;
  AD_CHECK(ad_linear_bwd(dt, (uint32_t)x.batch_size(), (uint32_t)in_, (uint32_t)out_, x.base_dptr(), kd.val.get(txn, id()).dptr(),
                         dy.base_dptr(), dxp, dw, db, mode == 1 ? 1 : 0, 1, conn.stream()));
}

// ------------------------------------------------------------------ bilinear upsample of a strip
vector<ActVar> UpsampleBilinear2DOpF::MakeParallel(size_t scale, vector<ActVar> inputs, shared_ptr<Context> ctx) {
  vector<ActVar> out;
  for (auto& x : inputs) out.push_back(make_shared<UpsampleBilinear2DOpF>(scale, num_ranks_of(ctx, inputs.size()), x, ctx));
  return out;
}
UpsampleBilinear2DOpF::UpsampleBilinear2DOpF(size_t scale, size_t num_ranks, ActVar x, shared_ptr<Context> ctx)
    : ActOp(x->rank(), ctx), x_(x), scale_(scale), num_ranks_(num_ranks) {
  inputs_.push_back(x);
  Shape3D d = x->shape();
  alloc_output(Shape3D(d.shape[0] * scale, d.shape[1] * scale, d.shape[2]), 0, 0, x->batch_shape());
}
// all rows of the (halo-padded) buffer, interior columns only
ad_tensor4 UpsampleBilinear2DOpF::low_view(Act& a) const {
  ad_tensor4 v = a.view_base();
  v.base = (char*)v.base + (long long)a.offset().shape[0] * v.sx * (long long)a.elem_size();
  v.W = (uint32_t)a.dim().shape[0];
  return v;
}
void UpsampleBilinear2DOpF::_forward(TxnId txn) {
  if (!y_.val.overwrite(txn, id())) return;
  GPUConn conn = gpu()->conn();
  Act& x = x_->data().val.get(txn, id());
  const size_t p = x.offset().shape[1], h = x.dim().shape[1];
  assert((p >= 1 || num_ranks_ == 1) && "a partitioned upsample reads one halo row of each neighbour");
  ad_tensor4 xv = low_view(x), yv = y_.val.get_excl(txn, id()).view_interior();
  AD_CHECK(ad_upsample_bilinear_fwd(&xv, &yv, (uint32_t)scale_, (int32_t)(rank_ * h) - (int32_t)p, (uint32_t)(h * num_ranks_),
                                    (uint32_t)(rank_ * h * scale_), conn.stream()));
}
void UpsampleBilinear2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  // every interior column of every row (halo rows included) is written; the zero pad columns of a
  // gradient buffer are never read
  const int mode = xd.grad.accumulate_full(txn, id(), always, zero_init(gpu()));
  if (!mode) return;
  GPUConn conn = gpu()->conn();
  Act& dx = xd.grad.get_mut(txn, id());
  const size_t p = dx.offset().shape[1], h = dx.dim().shape[1];
  ad_tensor4 dxv = low_view(dx), dyv = y_.grad.get(txn, id()).view_interior();
  AD_CHECK(ad_upsample_bilinear_bwd(&dyv, &dxv, (uint32_t)scale_, (int32_t)(rank_ * h) - (int32_t)p, (uint32_t)(h * num_ranks_),
                                    (uint32_t)(rank_ * h * scale_), mode == 1 ? 1 : 0, conn.stream()));
}

// ------------------------------------------------------------------ per-pixel softmax + NLL (sink)
vector<shared_ptr<CudnnSoftmaxNLLLoss2DOpF>> CudnnSoftmaxNLLLoss2DOpF::MakeParallel(vector<ActVar> logits, shared_ptr<Context> ctx) {
  vector<shared_ptr<CudnnSoftmaxNLLLoss2DOpF>> out;
  for (auto& x : logits) out.push_back(make_shared<CudnnSoftmaxNLLLoss2DOpF>(x, ctx));
  return out;
}
CudnnSoftmaxNLLLoss2DOpF::CudnnSoftmaxNLLLoss2DOpF(ActVar x, shared_ptr<Context> ctx) : x_(x), ctx_(ctx) {
  inputs_.push_back(x);
  Shape3D d = x->shape();
  n_ = x->batch_shape(); hw_ = d.shape[0] * d.shape[1]; classes_ = d.shape[2];
  GPUContext* g = gpu_of(ctx_, x_->rank());
  GPUConn conn = g->conn();
  labels_ = (uint32_t*)g->arena().alloc(n_ * hw_ * sizeof(uint32_t));
  loss_ = (float*)g->arena().alloc(n_ * hw_ * sizeof(float));
  dloss_ = (float*)g->arena().alloc(n_ * hw_ * sizeof(float));
  AD_CHECK(ad_fill_zero(labels_, n_ * hw_ * sizeof(uint32_t), conn.stream()));
  AD_CHECK(ad_fill_zero(loss_, n_ * hw_ * sizeof(float), conn.stream()));
  AD_CHECK(ad_array_set_constant(n_ * hw_, 1.0f, dloss_, conn.stream()));
  conn.sync();
}
size_t CudnnSoftmaxNLLLoss2DOpF::_load_val(TxnId, VarIdSet& vars, size_t offset, any* reader) {
  if (!vars.mask(label_var_)) return offset;
  if (reader) {
    const uint32_t* host = nullptr;
    if (auto sp = std::any_cast<Slice<uint32_t>>(reader)) host = sp->ptr;
    else if (auto hp = std::any_cast<uint32_t*>(reader)) host = *hp;
    assert(host && "labels are read from uint32_t* or Slice<uint32_t>");
    load_labels(host + (replica_ ? 0 : offset));
  }
  return replica_ ? offset : offset + n_ * hw_;
}
size_t CudnnSoftmaxNLLLoss2DOpF::_store_val(TxnId, VarIdSet& vars, size_t offset, any* writer) {
  if (!vars.mask(loss_var_)) return offset;
  if (replica_) return offset;
  if (writer) {
    float* host = host_floats(writer);
    assert(host);
    store_loss(host + offset);
  }
  return offset + n_ * hw_;
}
void CudnnSoftmaxNLLLoss2DOpF::load_labels(const uint32_t* host) {
  GPUConn conn = gpu_of(ctx_, x_->rank())->conn();
  CUDA_CHECK(cudaMemcpyAsync(labels_, host, n_ * hw_ * sizeof(uint32_t), cudaMemcpyHostToDevice, conn.stream()));
  conn.sync();
}
void CudnnSoftmaxNLLLoss2DOpF::set_loss_weight(float w) {
  GPUConn conn = gpu_of(ctx_, x_->rank())->conn();
  AD_CHECK(ad_array_set_constant(n_ * hw_, w, dloss_, conn.stream()));
  conn.sync();
}
void CudnnSoftmaxNLLLoss2DOpF::store_loss(float* host) {
  GPUConn conn = gpu_of(ctx_, x_->rank())->conn();
  CUDA_CHECK(cudaMemcpyAsync(host, loss_, n_ * hw_ * sizeof(float), cudaMemcpyDeviceToHost, conn.stream()));
  conn.sync();
}
double CudnnSoftmaxNLLLoss2DOpF::loss_sum() {
  // summed on the device by the two-stage statistics reduction (fixed order; fp32 partial sums of a few dozen terms,
  // combined in double) over the losses viewed as a one-channel tensor
  GPUContext* g = gpu_of(ctx_, x_->rank());
  GPUConn conn = g->conn();
  if (!loss_sum_dev_) loss_sum_dev_ = (float*)g->arena().alloc(64);
  g->reserve_scratch(ad_bn_scratch_bytes(1));
  ad_tensor4 t = {loss_, AD_F32, (uint32_t)n_, 1u, 1u, (uint32_t)hw_, (long long)hw_, (long long)hw_, (long long)hw_, 1};
  AD_CHECK(ad_bn_partial_stats(&t, loss_sum_dev_, g->get_scratch(), g->scratch_size(), conn.stream()));
  float h[2] = {0.f, 0.f};
  CUDA_CHECK(cudaMemcpyAsync(h, loss_sum_dev_, sizeof h, cudaMemcpyDeviceToHost, conn.stream()));
  conn.sync();
  return (double)h[0];
}
void CudnnSoftmaxNLLLoss2DOpF::_forward(TxnId txn) {
  GPUConn conn = gpu_of(ctx_, x_->rank())->conn();
  Act& x = x_->data().val.get(txn, id());
  assert(x.offset().shape[0] == 0 && x.offset().shape[1] == 0 && "the loss reads dense logits");
  const bool f32 = x.storage() == COMPUTE_F32_NCHW;
  AD_CHECK(ad_softmax_ce_pixel_fwd(f32 ? AD_F32 : AD_BF16, f32 ? AD_NCHW : AD_NHWC, (uint32_t)n_, (uint32_t)classes_, (uint32_t)hw_,
                                   x.base_dptr(), labels_, loss_, nullptr, conn.stream()));
}
void CudnnSoftmaxNLLLoss2DOpF::_backward(TxnId txn) {
  auto xd = x_->data();
  GPUContext* g = gpu_of(ctx_, x_->rank());
  const int mode = xd.grad.accumulate_full(txn, id(), unpadded, zero_init(g));
  if (!mode) return;
  GPUConn conn = g->conn();
  Act& x = xd.val.get(txn, id());
  Act& dx = xd.grad.get_mut(txn, id());
  const bool f32 = x.storage() == COMPUTE_F32_NCHW;
  AD_CHECK(ad_softmax_ce_pixel_bwd(f32 ? AD_F32 : AD_BF16, f32 ? AD_NCHW : AD_NHWC, (uint32_t)n_, (uint32_t)classes_, (uint32_t)hw_,
                                   x.base_dptr(), labels_, dloss_, dx.base_dptr(), mode == 1 ? 1 : 0, conn.stream()));
}

}  // namespace arraydiff
