// Device arrays of the op-graph API: GPUMemory, GPUArray{0,1,4}D, GPUBatchArray{0,1,3}D.
// Same roles as the reference's include/arraydiff/array_gpu.hh:67-689:
//   * dims are minor-first (Shape3D(w,h,c)); a batch array carries dim / offset / stride / batch;
//   * a padded activation allocates its whole padded extent zeroed; as_view() is the interior,
//     base_as_view() the padded origin (reference :508-548);
//   * memory comes from the rank's arena and is never freed (reference :82-109).
// Added: a storage tag.  An activation is logically fp32 but is stored either as NCHW fp32 (the
// reference's layout) or as NHWC bf16 (what the tensor-core kernels read), chosen by the context's
// ComputeMode when the array is created; host transfers always speak NCHW fp32.
#ifndef ARRAYDIFF_ARRAY_GPU_HH
#define ARRAYDIFF_ARRAY_GPU_HH

#include <cassert>
#include <cstring>
#include <vector>

#include "arraydiff/array_abstract.hh"
#include "arraydiff/context.hh"

namespace arraydiff {

#define AD_CHECK(call) do { int _st = (call); if (_st != AD_OK) ::arraydiff::ad_fail(_st, #call, __FILE__, __LINE__); } while (0)
#define CUDA_CHECK(call) do { cudaError_t _e = (call); if (_e != cudaSuccess) ::arraydiff::cuda_fail((int)_e, #call, __FILE__, __LINE__); } while (0)
[[noreturn]] void ad_fail(int status, const char* what, const char* file, int line);
[[noreturn]] void cuda_fail(int err, const char* what, const char* file, int line);

template <typename T>
class GPUMemory {
public:
  GPUMemory() : dptr_(nullptr), size_(0) {}
  GPUMemory(size_t size, GPUContext* ctx) : size_(size) {
    GPUConn conn = ctx->conn();
    dptr_ = (T*)ctx->arena().alloc(size * sizeof(T));
    AD_CHECK(ad_fill_zero(dptr_, size * sizeof(T), conn.stream()));
  }
  static GPUMemory<T> Zeros(size_t size, GPUContext* ctx) { return GPUMemory<T>(size, ctx); }
  T* dptr() const { return dptr_; }
  size_t size() const { return size_; }
  void set_constant(float c, GPUConn& conn);  // float only
  void load_sync(const T* src, size_t n, size_t dst_off, GPUConn& conn) {
    CUDA_CHECK(cudaMemcpyAsync(dptr_ + dst_off, src, n * sizeof(T), cudaMemcpyHostToDevice, conn.stream()));
    conn.sync();
  }
  void store_sync(T* dst, size_t n, size_t src_off, GPUConn& conn) const {
    CUDA_CHECK(cudaMemcpyAsync(dst, dptr_ + src_off, n * sizeof(T), cudaMemcpyDeviceToHost, conn.stream()));
    conn.sync();
  }
  void copy(const GPUMemory<T>& src, size_t n, size_t src_off, size_t dst_off, GPUConn& conn) {
    CUDA_CHECK(cudaMemcpyAsync(dptr_ + dst_off, src.dptr_ + src_off, n * sizeof(T), cudaMemcpyDeviceToDevice, conn.stream()));
  }
  // y = alpha * x + beta * y  (reference: array_gpu.hh add_scaled -> src/kernels/array.cu:96-109)
  void add_scaled(float alpha, const GPUMemory<T>& x, float beta, size_t n, size_t x_off, size_t y_off, GPUConn& conn) {
    AD_CHECK(ad_array_add_scaled(n, alpha, beta, x.dptr_ + x_off, dptr_ + y_off, conn.stream()));
  }
private:
  T* dptr_;
  size_t size_;
};

// Parameter-like arrays (filters Shape4D(kw,kh,c,k) = KCRS in memory; per-channel vectors).
template <typename ShapeT, typename T>
class GPUArrayND {
public:
  typedef ShapeT Shape;
  GPUArrayND() {}
  GPUArrayND(ShapeT dim, GPUContext* ctx) : dim_(dim), mem_(dim.flat_size() ? dim.flat_size() : 1, ctx) {}
  static GPUArrayND Zeros(ShapeT dim, GPUContext* ctx) { return GPUArrayND(dim, ctx); }
  static GPUArrayND ZerosPadded(ShapeT dim, ShapeT, ShapeT, GPUContext* ctx) { return GPUArrayND(dim, ctx); }
  ShapeT dim() const { return dim_; }
  size_t flat_size() const { return dim_.flat_size() ? dim_.flat_size() : 1; }
  T* dptr() const { return mem_.dptr(); }
  GPUMemory<T>& mem() { return mem_; }
private:
  ShapeT dim_;
  GPUMemory<T> mem_;
};
template <typename T> using GPUArray0D = GPUArrayND<Shape0D, T>;
template <typename T> using GPUArray1D = GPUArrayND<Shape1D, T>;
template <typename T> using GPUArray4D = GPUArrayND<Shape4D, T>;

// Activations: [batch][c][h][w] logically; (w,h,c) dims, optional halo padding.
template <typename T>
class GPUBatchArray3D {
public:
  typedef Shape3D Shape;
  GPUBatchArray3D() : batch_cap_(0), batch_(0), dptr_(nullptr), storage_(COMPUTE_F32_NCHW) {}
  // dim: interior dims; offset: (pw, ph, 0); stride: packed stride of the padded dims, i.e.
  // (1, W+2pw, (W+2pw)(H+2ph)) -- the reference's convention (src/op.cc:2556-2571).
  static GPUBatchArray3D ZerosPadded(Shape3D dim, Shape3D offset, Shape3D stride, size_t batch, GPUContext* ctx);
  static GPUBatchArray3D Zeros(Shape3D dim, size_t batch, GPUContext* ctx) {
    return ZerosPadded(dim, Shape3D(0, 0, 0), dim.packed_stride(), batch, ctx);
  }
  Shape3D dim() const { return dim_; }
  Shape3D offset() const { return offset_; }
  Shape3D stride() const { return stride_; }
  Shape3D padded_dim() const { return Shape3D(dim_.shape[0] + 2 * offset_.shape[0], dim_.shape[1] + 2 * offset_.shape[1], dim_.shape[2]); }
  size_t batch_capacity() const { return batch_cap_; }
  size_t batch_size() const { return batch_; }
  void set_batch_size(size_t b) { assert(b <= batch_cap_); batch_ = b; }
  ComputeMode storage() const { return storage_; }
  size_t elem_size() const { return storage_ == COMPUTE_F32_NCHW ? 4 : 2; }
  size_t padded_elems() const { return padded_dim().flat_size() * batch_cap_; }
  void* base_dptr() const { return dptr_; }                 // padded origin (base_as_view().dptr())
  void* interior_dptr() const;                               // interior origin (as_view().dptr())
  ad_tensor4 view_interior() const;                          // strided view of the interior
  ad_tensor4 view_base() const;                              // strided view of the whole padded extent
  void zero(GPUConn& conn) const { AD_CHECK(ad_fill_zero(dptr_, padded_elems() * elem_size(), conn.stream())); }
  // Host transfers in the reference's layout: packed NCHW fp32 of the INTERIOR.
  void load_host_nchw(const float* src, GPUContext* ctx) const;
  // rows [row0, row0 + h) of a packed NCHW fp32 host tensor of full_h rows: one pitched copy, so that a rank
  // receives its strip and nothing else
  void load_host_nchw_rows(const float* src_full, size_t full_h, size_t row0, GPUContext* ctx) const;
  // rows [row0, row0 + h) of a batch of full_h-row images stored [image][row][column][channel] fp32 on the host, every
  // element multiplied by `scale` on the way in
  void load_host_nhwc_rows(const T* src_full, size_t full_h, size_t row0, float scale, GPUContext* ctx) const;
  void store_host_nchw(float* dst, GPUContext* ctx) const;
private:
  Shape3D dim_, offset_, stride_;
  size_t batch_cap_, batch_;
  void* dptr_;
  ComputeMode storage_;
};

// Small batch arrays for losses / labels: [batch][d] and [batch].
template <typename T>
class GPUBatchArray1D {
public:
  typedef Shape1D Shape;
  GPUBatchArray1D() : batch_(0) {}
  static GPUBatchArray1D ZerosPadded(Shape1D dim, Shape1D, Shape1D, size_t batch, GPUContext* ctx) {
    GPUBatchArray1D a; a.dim_ = dim; a.batch_ = batch; a.mem_ = GPUMemory<T>(dim.flat_size() * batch, ctx); return a;
  }
  Shape1D dim() const { return dim_; }
  size_t batch_size() const { return batch_; }
  T* dptr() const { return mem_.dptr(); }
  GPUMemory<T>& mem() { return mem_; }
private:
  Shape1D dim_; size_t batch_; GPUMemory<T> mem_;
};
template <typename T>
class GPUBatchArray0D {
public:
  typedef Shape0D Shape;
  GPUBatchArray0D() : batch_(0) {}
  static GPUBatchArray0D ZerosPadded(Shape0D, Shape0D, Shape0D, size_t batch, GPUContext* ctx) {
    GPUBatchArray0D a; a.batch_ = batch; a.mem_ = GPUMemory<T>(batch, ctx); return a;
  }
  size_t batch_size() const { return batch_; }
  T* dptr() const { return mem_.dptr(); }
  GPUMemory<T>& mem() { return mem_; }
private:
  size_t batch_; GPUMemory<T> mem_;
};

}  // namespace arraydiff
#endif
