// Shapes of the op-graph API.  As in the reference (include/arraydiff/array_abstract.hh:93-166)
// every shape is MINOR-FIRST: Shape3D(w, h, c), Shape4D(kw, kh, c_in, c_out); index 0 is the
// fastest-varying axis of a packed array.
#ifndef ARRAYDIFF_ARRAY_ABSTRACT_HH
#define ARRAYDIFF_ARRAY_ABSTRACT_HH

#include <array>
#include <cstddef>
#include <initializer_list>

namespace arraydiff {

template <size_t D>
class ShapeND {
public:
  static ShapeND Zero() { return ShapeND(); }
  ShapeND() { shape.fill(0); }
  ShapeND(std::initializer_list<size_t> dims) {
    shape.fill(0);
    size_t i = 0;
    for (size_t d : dims) if (i < D) shape[i++] = d;
  }
  size_t major() const { return D ? shape[0] : 1; }
  size_t minor() const { return D ? shape[D - 1] : 1; }
  size_t flat_size() const {
    size_t n = 1;
    for (size_t i = 0; i < D; ++i) n *= shape[i];
    return n;
  }
  // stride of a packed array with these dims: (1, d0, d0*d1, ...)
  ShapeND packed_stride() const {
    ShapeND s;
    size_t acc = 1;
    for (size_t i = 0; i < D; ++i) { s.shape[i] = acc; acc *= shape[i]; }
    return s;
  }
  bool is_packed(const ShapeND& stride) const { return packed_stride().shape == stride.shape; }
  bool is_zero() const {
    for (size_t i = 0; i < D; ++i) if (shape[i]) return false;
    return true;
  }
  // this = index, stride = element strides -> flat element offset
  size_t to_index(const ShapeND& stride) const {
    size_t n = 0;
    for (size_t i = 0; i < D; ++i) n += shape[i] * stride.shape[i];
    return n;
  }
  bool operator==(const ShapeND& o) const { return shape == o.shape; }
  bool operator!=(const ShapeND& o) const { return !(shape == o.shape); }
  std::array<size_t, D> shape;
};

class Shape0D : public ShapeND<0> { public: Shape0D() {} };
class Shape1D : public ShapeND<1> { public: Shape1D() {} Shape1D(size_t d0) : ShapeND<1>({d0}) {} Shape1D(const ShapeND<1>& s) : ShapeND<1>(s) {} };
class Shape2D : public ShapeND<2> { public: Shape2D() {} Shape2D(size_t d0, size_t d1) : ShapeND<2>({d0, d1}) {} Shape2D(const ShapeND<2>& s) : ShapeND<2>(s) {} };
class Shape3D : public ShapeND<3> { public: Shape3D() {} Shape3D(size_t d0, size_t d1, size_t d2) : ShapeND<3>({d0, d1, d2}) {} Shape3D(const ShapeND<3>& s) : ShapeND<3>(s) {} };
class Shape4D : public ShapeND<4> { public: Shape4D() {} Shape4D(size_t d0, size_t d1, size_t d2, size_t d3) : ShapeND<4>({d0, d1, d2, d3}) {} Shape4D(const ShapeND<4>& s) : ShapeND<4>(s) {} };

}  // namespace arraydiff
#endif
