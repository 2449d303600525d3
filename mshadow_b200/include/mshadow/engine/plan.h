/*
 * Execution plans: the value-type mirror of an expression tree that a kernel receives as
 * its argument.  Plan<E,DType>::Eval(y, x) yields the element at row y / column x of the
 * expression viewed as a matrix (all leading dimensions folded into y), the contract that
 * dmlc/mshadow's mshadow/expr_engine-inl.h (:39-232) establishes and that user-defined
 * extension expressions rely on.
 *
 * New here: plans of element-wise nodes also expose EvalPack(y, x), which yields the 16-byte
 * group of elements starting at an x that is a multiple of the group width.  Tensor leaves
 * serve it with one 128-bit load, so a whole expression is evaluated on 128-bit coalesced
 * HBM accesses whatever user functors it contains.  Which expressions may take that path
 * is decided by the traits in engine/check.h.
 */
#ifndef MSHADOW_ENGINE_PLAN_H_
#define MSHADOW_ENGINE_PLAN_H_

#include "../base.h"
#include "../expression.h"

namespace mshadow {
template <typename Device, int dimension, typename DType>
struct Tensor;

namespace expr {

/*! \brief sixteen bytes worth of elements, the unit of vectorised memory access */
template <typename DType>
struct alignas(16) Pack {
  static const int kLanes = 16 / sizeof(DType);
  DType v[kLanes];
};

namespace plandetail {
#ifdef __CUDACC__
/*! \brief 128-bit streaming load; the data is not expected to be re-read soon */
template <typename DType>
__device__ __forceinline__ Pack<DType> LoadStream(const DType *p) {
  Pack<DType> r;
  *reinterpret_cast<int4 *>(&r) = __ldcs(reinterpret_cast<const int4 *>(p));
  return r;
}
/*! \brief 128-bit load through the regular cache path (small, re-used operands) */
template <typename DType>
__device__ __forceinline__ Pack<DType> LoadCached(const DType *p) {
  Pack<DType> r;
  *reinterpret_cast<int4 *>(&r) = *reinterpret_cast<const int4 *>(p);
  return r;
}
template <typename DType>
__device__ __forceinline__ void StoreStream(DType *p, const Pack<DType> &v) {
  __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&v));
}
#endif

/*
 * Checked build (-DMSHADOW_B200_CHECK_BOUNDS=1), the stand-in for a memory checker while
 * developing an expression plan: every access that a tensor leaf serves on the GPU is compared
 * with the extent of the tensor's storage.  An access outside it is not performed: a load yields
 * zero, a store is dropped, the first offending offset is recorded, and the kernel carries on,
 * so the context stays usable and nothing faults.  gpu_rt::TakeBoundsViolation() reads and clears
 * the record.  The record lives once per translation unit.  Off by default: the checks cost a
 * compare per access and 8 bytes per leaf in the kernel arguments.
 */
#ifndef MSHADOW_B200_CHECK_BOUNDS
#define MSHADOW_B200_CHECK_BOUNDS 0
#endif
#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDACC__)
struct BoundsRecord {
  int hit;                 // 0: clean
  int width;               // elements of the refused access
  long long offset, limit;  // element offset from the tensor's base, and the storage extent
};
static __device__ BoundsRecord g_bounds_record;
static __device__ long long g_bounds_sink[2];  // where refused l-value references point
static __device__ long long g_bounds_zero[2];  // what refused loads read (never written: all-zero bits)
__device__ __forceinline__ bool BoundsOk(long long offset, int width, long long limit) {
  if (offset >= 0 && offset + width <= limit) return true;
  if (atomicCAS(&g_bounds_record.hit, 0, 1) == 0) {
    g_bounds_record.width = width;
    g_bounds_record.offset = offset;
    g_bounds_record.limit = limit;
  }
  return false;
}
template <typename DType>
__device__ __forceinline__ DType &BoundsSink() {
  return *reinterpret_cast<DType *>(g_bounds_sink);
}
template <typename DType>
__device__ __forceinline__ const DType &BoundsZero() {
  return *reinterpret_cast<const DType *>(g_bounds_zero);
}
#endif
}  // namespace plandetail

/*!
 * \brief base of extension expressions that behave like a tensor of known shape
 *  (pooling, broadcasting, slicing...).  Same role and members as the reference's
 *  MakeTensorExp (mshadow/expr_engine-inl.h:24-34).
 */
template <typename SubType, typename SrcExp, int dim, typename DType>
struct MakeTensorExp : public Exp<MakeTensorExp<SubType, SrcExp, dim, DType>, DType, type::kChainer> {
  Shape<dim> shape_;
  inline const SubType &real_self() const { return *static_cast<const SubType *>(this); }
};

/*! \brief primary template: every expression type specialises this */
template <typename ExpType, typename DType>
class Plan {
 public:
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const;
};

// ---- an extension expression seen through its MakeTensorExp base (that is the type the
//      operators deduce for it): forwards to the plan of the real expression ----
template <typename SubType, typename SrcExp, int dim, typename DType>
class Plan<MakeTensorExp<SubType, SrcExp, dim, DType>, DType> {
 public:
  Plan(const Plan<SubType, DType> &real) : real_(real) {}  // NOLINT(*) implicit on purpose
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const { return real_.Eval(y, x); }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const { return real_.EvalPack(y, x); }
#endif

 private:
  Plan<SubType, DType> real_;
};

// ---- tensor leaf ----
#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDA_ARCH__)
#define MSHADOW_B200_BOUNDS_(offset, width, refused) \
  if (!plandetail::BoundsOk(offset, width, limit_)) refused
#else
#define MSHADOW_B200_BOUNDS_(offset, width, refused)
#endif

template <typename Device, int dim, typename DType>
class Plan<Tensor<Device, dim, DType>, DType> {
 public:
  explicit Plan(const Tensor<Device, dim, DType> &t) : dptr_(t.dptr_), stride_(t.stride_) {
#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDACC__)
    const Shape<2> flat = t.shape_.FlatTo2D();  // storage runs to the end of the last row
    limit_ = flat[0] == 0 ? 0 : static_cast<long long>(flat[0] - 1) * t.stride_ + flat[1];
#endif
  }
  MSHADOW_XINLINE DType &REval(index_t y, index_t x) {
    MSHADOW_B200_BOUNDS_(Offset(y, x), 1, return plandetail::BoundsSink<DType>());
    return dptr_[Offset(y, x)];
  }
  MSHADOW_XINLINE const DType &Eval(index_t y, index_t x) const {
    MSHADOW_B200_BOUNDS_(Offset(y, x), 1, return plandetail::BoundsZero<DType>());
    return dptr_[Offset(y, x)];
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    MSHADOW_B200_BOUNDS_(Offset(y, x), Pack<DType>::kLanes, return Pack<DType>());
    return plandetail::LoadStream(dptr_ + Offset(y, x));
  }
  __device__ __forceinline__ void StorePack(index_t y, index_t x, const Pack<DType> &v) {
    MSHADOW_B200_BOUNDS_(Offset(y, x), Pack<DType>::kLanes, return);
    plandetail::StoreStream(dptr_ + Offset(y, x), v);
  }
#endif
  /*! \brief re-interpret dense storage as rows of `width` elements */
  inline void Reflow(index_t width) { stride_ = width; }

 private:
  MSHADOW_XINLINE int64_t Offset(index_t y, index_t x) const {
    return static_cast<int64_t>(y) * stride_ + x;
  }
  DType *dptr_;
  index_t stride_;
#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDACC__)
  long long limit_;
#endif
};

// ---- 1-d tensor leaf: a single row ----
template <typename Device, typename DType>
class Plan<Tensor<Device, 1, DType>, DType> {
 public:
  explicit Plan(const Tensor<Device, 1, DType> &t) : dptr_(t.dptr_) {
#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDACC__)
    limit_ = t.shape_[0];
#endif
  }
  MSHADOW_XINLINE DType &REval(index_t, index_t x) {
    MSHADOW_B200_BOUNDS_(x, 1, return plandetail::BoundsSink<DType>());
    return dptr_[x];
  }
  MSHADOW_XINLINE const DType &Eval(index_t, index_t x) const {
    MSHADOW_B200_BOUNDS_(x, 1, return plandetail::BoundsZero<DType>());
    return dptr_[x];
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t, index_t x) const {
    MSHADOW_B200_BOUNDS_(x, Pack<DType>::kLanes, return Pack<DType>());
    return plandetail::LoadStream(dptr_ + x);
  }
  /*! \brief cached variant for operands that every row re-reads (broadcast sources) */
  __device__ __forceinline__ Pack<DType> EvalPackCached(index_t x) const {
    MSHADOW_B200_BOUNDS_(x, Pack<DType>::kLanes, return Pack<DType>());
    return plandetail::LoadCached(dptr_ + x);
  }
  __device__ __forceinline__ void StorePack(index_t, index_t x, const Pack<DType> &v) {
    MSHADOW_B200_BOUNDS_(x, Pack<DType>::kLanes, return);
    plandetail::StoreStream(dptr_ + x, v);
  }
#endif
  inline void Reflow(index_t) {}

 private:
  DType *dptr_;
#if MSHADOW_B200_CHECK_BOUNDS && defined(__CUDACC__)
  long long limit_;
#endif
};

// ---- scalar ----
template <typename DType>
class Plan<ScalarExp<DType>, DType> {
 public:
  explicit Plan(DType scalar) : scalar_(scalar) {}
  MSHADOW_XINLINE DType Eval(index_t, index_t) const { return scalar_; }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t, index_t) const {
    Pack<DType> r;
#pragma unroll
    for (int i = 0; i < Pack<DType>::kLanes; ++i) r.v[i] = scalar_;
    return r;
  }
#endif
  inline void Reflow(index_t) {}

 private:
  DType scalar_;
};

// ---- type cast ----
template <typename DstDType, typename SrcDType, typename EType, int etype>
class Plan<TypecastExp<DstDType, SrcDType, EType, etype>, DstDType> {
 public:
  explicit Plan(const Plan<EType, SrcDType> &src) : src_(src) {}
  MSHADOW_XINLINE DstDType Eval(index_t y, index_t x) const {
    return static_cast<DstDType>(src_.Eval(y, x));
  }

 private:
  Plan<EType, SrcDType> src_;
};

// ---- element-wise maps ----
template <typename OP, typename TA, typename DType, int etype>
class Plan<UnaryMapExp<OP, TA, DType, etype>, DType> {
 public:
  explicit Plan(const Plan<TA, DType> &src) : src_(src) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const { return OP::Map(src_.Eval(y, x)); }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    Pack<DType> a = src_.EvalPack(y, x);
#pragma unroll
    for (int i = 0; i < Pack<DType>::kLanes; ++i) a.v[i] = OP::Map(a.v[i]);
    return a;
  }
#endif
  inline void Reflow(index_t w) { src_.Reflow(w); }

 private:
  Plan<TA, DType> src_;
};

template <typename OP, typename TA, typename TB, typename DType, int etype>
class Plan<BinaryMapExp<OP, TA, TB, DType, etype>, DType> {
 public:
  explicit Plan(const Plan<TA, DType> &lhs, const Plan<TB, DType> &rhs) : lhs_(lhs), rhs_(rhs) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    return OP::Map(lhs_.Eval(y, x), rhs_.Eval(y, x));
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    Pack<DType> a = lhs_.EvalPack(y, x);
    const Pack<DType> b = rhs_.EvalPack(y, x);
#pragma unroll
    for (int i = 0; i < Pack<DType>::kLanes; ++i) a.v[i] = OP::Map(a.v[i], b.v[i]);
    return a;
  }
#endif
  inline void Reflow(index_t w) {
    lhs_.Reflow(w);
    rhs_.Reflow(w);
  }

 private:
  Plan<TA, DType> lhs_;
  Plan<TB, DType> rhs_;
};

template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
class Plan<TernaryMapExp<OP, TA, TB, TC, DType, etype>, DType> {
 public:
  explicit Plan(const Plan<TA, DType> &i1, const Plan<TB, DType> &i2, const Plan<TC, DType> &i3)
      : item1_(i1), item2_(i2), item3_(i3) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const {
    return OP::Map(item1_.Eval(y, x), item2_.Eval(y, x), item3_.Eval(y, x));
  }
#ifdef __CUDACC__
  __device__ __forceinline__ Pack<DType> EvalPack(index_t y, index_t x) const {
    Pack<DType> a = item1_.EvalPack(y, x);
    const Pack<DType> b = item2_.EvalPack(y, x);
    const Pack<DType> c = item3_.EvalPack(y, x);
#pragma unroll
    for (int i = 0; i < Pack<DType>::kLanes; ++i) a.v[i] = OP::Map(a.v[i], b.v[i], c.v[i]);
    return a;
  }
#endif
  inline void Reflow(index_t w) {
    item1_.Reflow(w);
    item2_.Reflow(w);
    item3_.Reflow(w);
  }

 private:
  Plan<TA, DType> item1_;
  Plan<TB, DType> item2_;
  Plan<TC, DType> item3_;
};

// ---- transposed matrix ----
template <typename EType, typename DType>
class Plan<TransposeExp<EType, DType>, DType> {
 public:
  explicit Plan(const Plan<EType, DType> &src) : src_(src) {}
  MSHADOW_XINLINE DType Eval(index_t y, index_t x) const { return src_.Eval(x, y); }

 private:
  Plan<EType, DType> src_;
};

// ---- plan construction: one overload per node type, recursing into operands ----
template <typename OP, typename TA, typename DType, int etype>
inline Plan<UnaryMapExp<OP, TA, DType, etype>, DType> MakePlan(
    const UnaryMapExp<OP, TA, DType, etype> &e);
template <typename OP, typename TA, typename TB, typename DType, int etype>
inline Plan<BinaryMapExp<OP, TA, TB, DType, etype>, DType> MakePlan(
    const BinaryMapExp<OP, TA, TB, DType, etype> &e);
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
inline Plan<TernaryMapExp<OP, TA, TB, TC, DType, etype>, DType> MakePlan(
    const TernaryMapExp<OP, TA, TB, TC, DType, etype> &e);

template <typename DType>
inline Plan<ScalarExp<DType>, DType> MakePlan(const ScalarExp<DType> &e) {
  return Plan<ScalarExp<DType>, DType>(e.scalar_);
}
template <typename DstDType, typename SrcDType, typename EType, int etype>
inline Plan<TypecastExp<DstDType, SrcDType, EType, etype>, DstDType> MakePlan(
    const TypecastExp<DstDType, SrcDType, EType, etype> &e) {
  return Plan<TypecastExp<DstDType, SrcDType, EType, etype>, DstDType>(MakePlan(e.exp));
}
template <typename T, typename DType>
inline Plan<T, DType> MakePlan(const RValueExp<T, DType> &e) {
  return Plan<T, DType>(e.self());
}
template <typename T, typename DType>
inline Plan<TransposeExp<T, DType>, DType> MakePlan(const TransposeExp<T, DType> &e) {
  return Plan<TransposeExp<T, DType>, DType>(MakePlan(e.exp));
}
template <typename T, typename SrcExp, int dim, typename DType>
inline Plan<T, DType> MakePlan(const MakeTensorExp<T, SrcExp, dim, DType> &e) {
  return Plan<T, DType>(e.real_self());
}
template <typename OP, typename TA, typename DType, int etype>
inline Plan<UnaryMapExp<OP, TA, DType, etype>, DType> MakePlan(
    const UnaryMapExp<OP, TA, DType, etype> &e) {
  return Plan<UnaryMapExp<OP, TA, DType, etype>, DType>(MakePlan(e.src_));
}
template <typename OP, typename TA, typename TB, typename DType, int etype>
inline Plan<BinaryMapExp<OP, TA, TB, DType, etype>, DType> MakePlan(
    const BinaryMapExp<OP, TA, TB, DType, etype> &e) {
  return Plan<BinaryMapExp<OP, TA, TB, DType, etype>, DType>(MakePlan(e.lhs_), MakePlan(e.rhs_));
}
template <typename OP, typename TA, typename TB, typename TC, typename DType, int etype>
inline Plan<TernaryMapExp<OP, TA, TB, TC, DType, etype>, DType> MakePlan(
    const TernaryMapExp<OP, TA, TB, TC, DType, etype> &e) {
  return Plan<TernaryMapExp<OP, TA, TB, TC, DType, etype>, DType>(
      MakePlan(e.item1_), MakePlan(e.item2_), MakePlan(e.item3_));
}

}  // namespace expr
}  // namespace mshadow
#endif  // MSHADOW_ENGINE_PLAN_H_
