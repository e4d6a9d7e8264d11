// A synthetic data source for training drivers: `size` items of width x height x channels values with label
// index % num_labels -- the stand-in the reference provides for its ImageNet pipeline
// (include/arraydiff/io/dummy.hh:14-38; MutDatum: include/arraydiff/io/pipeline.hh).  The reference leaves the
// buffer uninitialised; here item `index` is filled with reproducible pseudo-random values in [0, 255], offset by
// its label so that a classifier has something to learn.
#ifndef ARRAYDIFF_IO_DUMMY_HH
#define ARRAYDIFF_IO_DUMMY_HH

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <utility>

namespace arraydiff {
namespace io {

using std::make_pair;
using std::pair;

template <typename T>
class MutDatum {
public:
  static MutDatum<T> Alloc(size_t size) { return MutDatum<T>{(T*)std::malloc(sizeof(T) * size), size}; }
  void dealloc() { std::free(buffer); buffer = nullptr; size = 0; }
  T* buffer;
  size_t size;
};

template <typename T>
class DummyData {
public:
  DummyData(size_t width, size_t height, size_t channels, uint32_t num_labels, size_t size)
      : width_(width), height_(height), channels_(channels), num_labels_(num_labels), size_(size) {}
  size_t size() const { return size_; }
  pair<MutDatum<T>, uint32_t> at(size_t index) const {
    auto datum = MutDatum<T>::Alloc(width_ * height_ * channels_);
    const uint32_t label = (uint32_t)(index % num_labels_);
    uint64_t s = 0x9E3779B97F4A7C15ull * (uint64_t)(index + 1);
    const float shift = 96.0f * (float)label / (float)num_labels_;
    for (size_t i = 0; i < datum.size; ++i) {
      s ^= s << 13; s ^= s >> 7; s ^= s << 17;                 // xorshift64
      datum.buffer[i] = (T)(shift + (float)(s >> 40) * (159.0f / 16777216.0f));
    }
    return make_pair(datum, label);
  }
private:
  size_t width_, height_, channels_;
  uint32_t num_labels_;
  size_t size_;
};

}  // namespace io
}  // namespace arraydiff
#endif
