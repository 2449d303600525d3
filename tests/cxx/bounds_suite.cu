/*
 * The checked build of the engine (-DMSHADOW_B200_CHECK_BOUNDS=1) on deliberately wrong
 * user-written expression plans: accesses beyond a tensor's storage must be refused (loads read
 * zero, stores are dropped), recorded, and leave the device usable.  Nothing here touches memory
 * outside an allocation: that is the point of the build.  Test code only.
 */
#include <cstdint>
#include <string>
#include <vector>

#include "mshadow/tensor.h"

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

namespace {

// a user expression with an index bug: column x reads column x + shift of its source
template <typename SrcExp>
struct ShiftedExp : public MakeTensorExp<ShiftedExp<SrcExp>, SrcExp, 2, float> {
  const SrcExp &src_;
  index_t shift_;
  ShiftedExp(const SrcExp &src, index_t shift) : src_(src), shift_(shift) {
    this->shape_ = ShapeCheck<2, SrcExp>::Check(src_);
  }
};
template <typename SrcExp>
inline ShiftedExp<SrcExp> shifted(const Exp<SrcExp, float, type::kRValue> &src, index_t shift) {
  return ShiftedExp<SrcExp>(src.self(), shift);
}
// the same bug on the left of an assignment: column x of the target is column x + shift of the tensor
template <typename SrcExp>
struct ShiftedDst : public TRValue<ShiftedDst<SrcExp>, gpu, 2, float> {
  const SrcExp &src_;
  index_t shift_;
  Shape<2> shape_;
  ShiftedDst(const SrcExp &src, index_t shift) : src_(src), shift_(shift) { shape_ = ShapeCheck<2, SrcExp>::Check(src_); }
  template <typename E, int etype>
  inline void operator=(const Exp<E, float, etype> &exp) {
    this->__assign(exp);
  }
  inline void operator=(const float &scalar) { this->__assign(scalar); }
};
}  // namespace

namespace mshadow {
namespace expr {
template <typename SrcExp>
class Plan<ShiftedExp<SrcExp>, float> {
 public:
  explicit Plan(const ShiftedExp<SrcExp> &e) : src_(MakePlan(e.src_)), shift_(e.shift_) {}
  MSHADOW_XINLINE float Eval(index_t y, index_t x) const { return src_.Eval(y, x + shift_); }

 private:
  Plan<SrcExp, float> src_;
  index_t shift_;
};
template <typename SrcExp>
class Plan<ShiftedDst<SrcExp>, float> {
 public:
  explicit Plan(const ShiftedDst<SrcExp> &e) : src_(MakePlan(e.src_)), shift_(e.shift_) {}
  MSHADOW_XINLINE float Eval(index_t y, index_t x) const { return src_.Eval(y, x + shift_); }
  MSHADOW_XINLINE float &REval(index_t y, index_t x) { return src_.REval(y, x + shift_); }

 private:
  Plan<SrcExp, float> src_;
  index_t shift_;
};
template <typename SrcExp>
inline Plan<ShiftedDst<SrcExp>, float> MakePlan(const ShiftedDst<SrcExp> &e) {
  return Plan<ShiftedDst<SrcExp>, float>(e);
}
template <typename SrcExp>
struct ShapeCheck<2, ShiftedDst<SrcExp> > {
  inline static Shape<2> Check(const ShiftedDst<SrcExp> &t) { return t.shape_; }
};
template <typename SrcExp>
struct StreamInfo<gpu, ShiftedDst<SrcExp> > {
  inline static Stream<gpu> *Get(const ShiftedDst<SrcExp> &t) { return StreamInfo<gpu, SrcExp>::Get(t.src_); }
};
template <typename SrcExp>
struct ExpInfo<ShiftedDst<SrcExp> > {
  static const int kDim = 2;
  static const int kDevMask = ExpInfo<SrcExp>::kDevMask;
};
}  // namespace expr
}  // namespace mshadow

namespace {
std::string g_error;

/*
 * case 0  dst = A + 1                       correct: no record
 * case 1  dst = shifted(A, shift)           reads run past the end of A's storage in the last row(s)
 * case 2  ShiftedDst(dst, shift) = A         stores run past the end of dst's storage in the last row(s)
 * out receives dst (rows x cols, row-major); record = {hit, width, offset, limit}
 */
int Run(int id, const float *a, float *out, int rows, int cols, int shift, long long record[4]) {
  InitTensorEngine<gpu>(0);
  Stream<gpu> *st = NewStream<gpu>(0);
  Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, false, st);
  Tensor<gpu, 2, float> D = NewTensor<gpu>(Shape2(rows, cols), -1.0f, false, st);
  Tensor<cpu, 2, float> ha(const_cast<float *>(a), Shape2(rows, cols)), hout(out, Shape2(rows, cols));
  Copy(A, ha, st);
  switch (id) {
    case 0: D = A + 1.0f; break;
    case 1: D = shifted(A, shift); break;
    default: {
      ShiftedDst<Tensor<gpu, 2, float> > target(D, shift);
      target = A;
    } break;
  }
  long long offset = 0, limit = 0;
  int width = 0;
  const bool hit = gpu_rt::TakeBoundsViolation(&offset, &width, &limit);
  record[0] = hit;
  record[1] = width;
  record[2] = offset;
  record[3] = limit;
  Copy(hout, D, st);
  st->Wait();
  FreeSpace(&A);
  FreeSpace(&D);
  DeleteStream(st);
  ShutdownTensorEngine<gpu>();
  return 0;
}
}  // namespace

extern "C" const char *msb_bounds_suite_error(void) { return g_error.c_str(); }

extern "C" int msb_bounds_suite_run(int id, const float *a, float *out, int rows, int cols, int shift,
                                    long long *record) {
  try {
    return Run(id, a, out, rows, cols, shift, record);
  } catch (const std::exception &e) {
    g_error = e.what();
    return -2;
  }
}
