// A borrowed host range: the reader / writer type the reference's tools hand to load_val / store_val
// (include/arraydiff/slice.hh:9-17; tools/train_imagenet.cc:216-243).
#ifndef ARRAYDIFF_SLICE_HH
#define ARRAYDIFF_SLICE_HH

#include <cstddef>

namespace arraydiff {

template <typename T>
class Slice {
public:
  Slice(T* ptr, size_t size) : ptr(ptr), size(size) {}
  T* ptr;
  size_t size;
};

}  // namespace arraydiff
#endif
