/*
 * Conformance programs for the header-level C++ API, in the style of the reference's own
 * GPU-vs-CPU checks (test/test.cu, guide/basic.cpp, guide/defop.cpp): each case is written
 * exactly as a user of dmlc/mshadow would write it against `mshadow/tensor.h`, runs on the
 * GPU, and hands its result back in a host buffer for the Python test to compare with a
 * numpy restatement.  Built into tests/cxx/libmsb_api_suite.so by mshadow_b200/build.py.
 */
#include <cmath>
#include <cstdio>
#include <vector>

#include "mshadow/tensor.h"
#include "mshadow/gpu/math.h"

using namespace mshadow;        // NOLINT(*)
using namespace mshadow::expr;  // NOLINT(*)

namespace {

// a user-defined operator, as in guide/defop.cpp
struct addone_square {
  MSHADOW_XINLINE static float Map(float a) {
    const float b = a + 1.0f;
    return b * b;
  }
};
struct maximum_op {
  MSHADOW_XINLINE static float Map(float a, float b) { return a > b ? a : b; }
};
// the same written for binary16 operands
struct maximum_half {
  MSHADOW_XINLINE static mshadow::half::half_t Map(mshadow::half::half_t a, mshadow::half::half_t b) { return a > b ? a : b; }
};

template <int dim>
void Upload(Tensor<gpu, dim, float> dst, const float *host, Stream<gpu> *s) {
  Tensor<cpu, dim, float> h(const_cast<float *>(host), dst.shape_);
  Copy(dst, h, s);
}
template <int dim>
void Download(float *host, Tensor<gpu, dim, float> src, Stream<gpu> *s) {
  Tensor<cpu, dim, float> h(host, src.shape_);
  Copy(h, src, s);
  s->Wait();
}

int RunCase(int id, const float *a, const float *b, float *out, int rows, int cols) {
  InitTensorEngine<gpu>(0);
  Stream<gpu> *st = NewStream<gpu>(0);
  int rc = 0;
  switch (id) {
    case 0: {  // pitched AllocSpace, TensorContainer, scalar on the right as an int literal
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      TensorContainer<gpu, 2, float> B(Shape2(rows, cols)), C;
      B.set_stream(st);
      C.set_stream(st);
      C.Resize(Shape2(rows, cols));
      Upload(A, a, st);
      Upload<2>(B, b, st);
      C = A + B * 2;
      Download<2>(out, C, st);
      out[rows * cols] = static_cast<float>(A.stride_);  // lets the test see the pitch
      FreeSpace(&A);
      break;
    }
    case 1: {  // scaled column sums, then accumulation into the same vector
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, float> B = NewTensor<gpu>(Shape2(rows, cols), 0.0f, false, st);
      Tensor<gpu, 1, float> v = NewTensor<gpu>(Shape1(cols), 0.0f, true, st);
      Upload(A, a, st);
      Upload(B, b, st);
      v = 0.5f * sum_rows(A);
      v += sum_rows(B);
      Download(out, v, st);
      FreeSpace(&A);
      FreeSpace(&B);
      FreeSpace(&v);
      break;
    }
    case 2: {  // test/test.cu: sumall_except_dim<0> of a 3-d tensor (rows = 3 * r1)
      const int r1 = rows / 3;
      Tensor<gpu, 3, float> A = NewTensor<gpu>(Shape3(3, r1, cols), 0.0f, true, st);
      Tensor<gpu, 1, float> v = NewTensor<gpu>(Shape1(3), 0.0f, true, st);
      Upload(A, a, st);
      v = sumall_except_dim<0>(A);
      Download(out, v, st);
      FreeSpace(&A);
      FreeSpace(&v);
      break;
    }
    case 3: {  // reduction over an expression, 4-d (2, rows/2, 2, cols/2), plusto
      Shape<4> s4 = Shape4(2, rows / 2, 2, cols / 2);
      Tensor<gpu, 4, float> A = NewTensor<gpu>(s4, 0.0f, false, st), B = NewTensor<gpu>(s4, 0.0f, false, st);
      Tensor<gpu, 1, float> v = NewTensor<gpu>(Shape1(rows / 2), 1.0f, true, st);
      Upload(A, a, st);
      Upload(B, b, st);
      v += sumall_except_dim<1>(A * B);
      Download(out, v, st);
      FreeSpace(&A);
      FreeSpace(&B);
      FreeSpace(&v);
      break;
    }
    case 4: {  // transposed operand
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, float> C = NewTensor<gpu>(Shape2(cols, rows), 0.0f, true, st);
      Upload(A, a, st);
      C = A.T() + 1.0f;
      Download(out, C, st);
      FreeSpace(&A);
      FreeSpace(&C);
      break;
    }
    case 5: {  // type casts: float -> int -> float
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, int> I = NewTensor<gpu>(Shape2(rows, cols), 0, true, st);
      Tensor<gpu, 2, float> C = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Upload(A, a, st);
      I = tcast<int>(A * 10.0f);
      I += 3;
      C = tcast<float>(I);
      Download(out, C, st);
      FreeSpace(&A);
      FreeSpace(&I);
      FreeSpace(&C);
      break;
    }
    case 6: {  // Slice and operator[]: rows 1..rows-2 get A + repmat(first row of B)
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, float> B = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, float> C = NewTensor<gpu>(Shape2(rows, cols), -1.0f, true, st);
      Upload(A, a, st);
      Upload(B, b, st);
      Tensor<gpu, 2, float> mid = C.Slice(1, rows - 1);
      mid = A.Slice(1, rows - 1) + repmat(B[0], rows - 2);
      Download(out, C, st);
      FreeSpace(&A);
      FreeSpace(&B);
      FreeSpace(&C);
      break;
    }
    case 7: {  // reduce_except_dim with the maximum reducer, and a binary user functor
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, float> B = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 1, float> v = NewTensor<gpu>(Shape1(cols), 0.0f, true, st);
      Upload(A, a, st);
      Upload(B, b, st);
      v = reduce_except_dim<1, red::maximum>(F<maximum_op>(A, B));
      Download(out, v, st);
      FreeSpace(&A);
      FreeSpace(&B);
      FreeSpace(&v);
      break;
    }
    case 8: {  // double precision goes through the same engine (two lanes per 16-byte group)
      Tensor<gpu, 2, double> A = NewTensor<gpu>(Shape2(rows, cols), 0.0, true, st);
      Tensor<gpu, 2, double> C = NewTensor<gpu>(Shape2(rows, cols), 0.0, true, st);
      std::vector<double> ha(static_cast<size_t>(rows) * cols), hc(ha.size());
      for (size_t i = 0; i < ha.size(); ++i) ha[i] = a[i];
      Copy(A, Tensor<cpu, 2, double>(ha.data(), A.shape_), st);
      C = A * A + 0.25;
      C /= A * 0.0 + 3.0;
      Copy(Tensor<cpu, 2, double>(hc.data(), C.shape_), C, st);
      st->Wait();
      for (size_t i = 0; i < hc.size(); ++i) out[i] = static_cast<float>(hc[i]);
      FreeSpace(&A);
      FreeSpace(&C);
      break;
    }
    case 9: {  // in place, unary user functor, guide/defop.cpp style
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Upload(A, a, st);
      A = F<addone_square>(A);
      A = F<b200::sigmoid>(A * 0.5f);
      Download(out, A, st);
      FreeSpace(&A);
      break;
    }
    case 10: {  // Softmax in place and SoftmaxGrad, labels = first column of b
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 1, float> lab = NewTensor<gpu>(Shape1(rows), 0.0f, true, st);
      Upload(A, a, st);
      std::vector<float> hl(rows);
      for (int i = 0; i < rows; ++i) hl[i] = b[static_cast<size_t>(i) * cols];
      Copy(lab, Tensor<cpu, 1, float>(hl.data(), Shape1(rows)), st);
      Softmax(A, A);
      SoftmaxGrad(A, A, lab);
      Download(out, A, st);
      FreeSpace(&A);
      FreeSpace(&lab);
      break;
    }
    case 11: {  // pooling over an expression: the window loop runs in the generic kernel
      Shape<4> s4 = Shape4(2, rows / 2, cols, cols);  // a holds 2 * (rows/2) images of cols x cols
      Tensor<gpu, 4, float> A = NewTensor<gpu>(s4, 0.0f, false, st);
      const int p = (cols - 3) / 2 + 1;
      Tensor<gpu, 4, float> P = NewTensor<gpu>(Shape4(2, rows / 2, p, p), 0.0f, false, st);
      Upload(A, a, st);
      P = pool<red::maximum>(A * 2.0f, 3, 3, 2, 2);
      Download(out, P, st);
      FreeSpace(&A);
      FreeSpace(&P);
      break;
    }
    case 12: {  // pool -> unpool -> chpool on plain tensors: the dedicated kernels
      Shape<4> s4 = Shape4(2, rows / 2, cols, cols);
      Tensor<gpu, 4, float> A = NewTensor<gpu>(s4, 0.0f, false, st), G = NewTensor<gpu>(s4, 0.0f, false, st);
      const int p = (cols - 3) / 2 + 1;
      Tensor<gpu, 4, float> P = NewTensor<gpu>(Shape4(2, rows / 2, p, p), 0.0f, false, st);
      Upload(A, a, st);
      P = pool<red::maximum>(A, 3, 3, 2, 2);
      G = unpool<red::maximum>(A, P, P, 3, 3, 2, 2);
      A = chpool<red::sum>(G, 3);
      Download(out, A, st);
      FreeSpace(&A);
      FreeSpace(&G);
      FreeSpace(&P);
      break;
    }
    case 13: {  // a shape mismatch is reported through CHECK
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, float> C = NewTensor<gpu>(Shape2(rows, cols + 1), 0.0f, true, st);
      try {
        C = A + 1.0f;
        rc = 1;  // must not get here
      } catch (const dmlc::Error &e) {
        rc = 100;
      }
      FreeSpace(&A);
      FreeSpace(&C);
      break;
    }
    case 14: {  // binary16 tensors: eight elements per 16-byte group, every operation rounded to half
      typedef mshadow::half::half_t H;
      const size_t n = static_cast<size_t>(rows) * cols;
      Tensor<gpu, 2, H> A = NewTensor<gpu>(Shape2(rows, cols), H(0.0f), true, st);
      Tensor<gpu, 2, H> B = NewTensor<gpu>(Shape2(rows, cols), H(0.0f), true, st);
      Tensor<gpu, 2, H> C = NewTensor<gpu>(Shape2(rows, cols), H(0.0f), true, st);
      std::vector<H> ha(n), hb(n), hc(n);
      for (size_t i = 0; i < n; ++i) ha[i] = H(a[i]), hb[i] = H(b[i]);
      Copy(A, Tensor<cpu, 2, H>(ha.data(), A.shape_), st);
      Copy(B, Tensor<cpu, 2, H>(hb.data(), B.shape_), st);
      C = A * B + A * H(0.5f) - B / (A * A + H(2.0f));  // scalars are written in the element type, as in the reference
      C += F<maximum_half>(A, B);
      Copy(Tensor<cpu, 2, H>(hc.data(), C.shape_), C, st);
      st->Wait();
      for (size_t i = 0; i < n; ++i) out[i] = static_cast<float>(hc[i]);
      FreeSpace(&A);
      FreeSpace(&B);
      FreeSpace(&C);
      break;
    }
    case 15: {  // casts between float and binary16 tensors, and a half reduction with an exact reducer
      typedef mshadow::half::half_t H;
      Tensor<gpu, 2, float> A = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 2, H> Ah = NewTensor<gpu>(Shape2(rows, cols), H(0.0f), true, st);
      Tensor<gpu, 2, float> C = NewTensor<gpu>(Shape2(rows, cols), 0.0f, true, st);
      Tensor<gpu, 1, H> colmax = NewTensor<gpu>(Shape1(cols), H(0.0f), true, st);
      Tensor<gpu, 1, float> colmax_f = NewTensor<gpu>(Shape1(cols), 0.0f, true, st);
      Upload(A, a, st);
      Ah = tcast<H>(A);
      C = tcast<float>(Ah) * 2.0f;
      colmax = reduce_except_dim<1, red::maximum>(Ah);
      colmax_f = tcast<float>(colmax);
      Download(out, C, st);
      Download(out + static_cast<size_t>(rows) * cols, colmax_f, st);
      FreeSpace(&A);
      FreeSpace(&Ah);
      FreeSpace(&C);
      FreeSpace(&colmax);
      FreeSpace(&colmax_f);
      break;
    }
    case 16: {  // guide/neuralnet/convnet.cu style: patches of a 3-d image to columns and back, accumulating savers
      const Shape<3> s3 = Shape3(2, 24, rows * cols / 48);
      Tensor<gpu, 3, float> A = NewTensor<gpu>(s3, 0.0f, false, st), G = NewTensor<gpu>(s3, 0.0f, false, st);
      Upload(A, a, st);
      Upload(G, b, st);
      const index_t oh = s3[1] - 2, ow = s3[2] - 2;
      Tensor<gpu, 2, float> M = NewTensor<gpu>(Shape2(3 * 3 * 2, oh * ow), 1.0f, false, st);
      M += unpack_patch2col(A, 3, 3, 1, 1);
      G -= pack_col2patch(M, G.shape_, 3, 3, 1, 1);
      const index_t oh2 = (s3[1] - 4) / 2 + 1, ow2 = s3[2] - 1;  // 4 x 2 patches, stride (2, 1)
      Tensor<gpu, 2, float> M2 = NewTensor<gpu>(Shape2(4 * 2 * 2, oh2 * ow2), 0.0f, false, st);
      M2 = unpack_patch2col(A, 4, 2, 2, 1, 1, 1);
      G += pack_col2patch(M2, G.shape_, 4, 2, 2, 1, 1, 1);
      Download(out, G, st);
      FreeSpace(&A);
      FreeSpace(&G);
      FreeSpace(&M);
      FreeSpace(&M2);
      break;
    }
    case 17: {  // the same round trip on pitched tensors (row pitch != width), 16-byte-aligned runs
      const Shape<3> s3 = Shape3(2, 12, 68);  // wide enough for AllocSpace to pitch the rows; out has one extra slot
      Tensor<gpu, 3, float> A = NewTensor<gpu>(s3, 0.0f, true, st), G = NewTensor<gpu>(s3, 0.0f, true, st);
      Tensor<cpu, 3, float> ha(const_cast<float *>(a), s3), hb(const_cast<float *>(b), s3), hout(out, s3);
      Copy(A, ha, st);
      Copy(G, hb, st);
      Tensor<gpu, 2, float> M = NewTensor<gpu>(Shape2(3 * 3 * 2, 10 * 66), 1.0f, true, st);
      M += unpack_patch2col(A, 3, 3, 1, 1);
      G -= pack_col2patch(M, G.shape_, 3, 3, 1, 1);
      Copy(hout, G, st);
      st->Wait();
      out[s3.Size()] = static_cast<float>(A.stride_ != s3[2]) + 2.0f * static_cast<float>(M.stride_ != M.size(1));
      FreeSpace(&A);
      FreeSpace(&G);
      FreeSpace(&M);
      break;
    }
    case 18: {  // the patch kernels are templates over the element type: binary64
      const Shape<3> s3 = Shape3(2, 24, 26);
      Tensor<gpu, 3, float> Af = NewTensor<gpu>(s3, 0.0f, false, st), Gf = NewTensor<gpu>(s3, 0.0f, false, st);
      Tensor<cpu, 3, float> ha(const_cast<float *>(a), s3), hb(const_cast<float *>(b), s3), hout(out, s3);
      Copy(Af, ha, st);
      Copy(Gf, hb, st);
      Tensor<gpu, 3, double> A = NewTensor<gpu>(s3, 0.0, false, st), G = NewTensor<gpu>(s3, 0.0, false, st);
      A = tcast<double>(Af);
      G = tcast<double>(Gf);
      Tensor<gpu, 2, double> M = NewTensor<gpu>(Shape2(3 * 3 * 2, 22 * 24), 0.0, false, st);
      M = unpack_patch2col(A, 3, 3, 1, 1);
      G += pack_col2patch(M, G.shape_, 3, 3, 1, 1);
      Gf = tcast<float>(G);
      Copy(hout, Gf, st);
      st->Wait();
      FreeSpace(&Af);
      FreeSpace(&Gf);
      FreeSpace(&A);
      FreeSpace(&G);
      FreeSpace(&M);
      break;
    }
    default:
      rc = -1;
  }
  st->Wait();
  DeleteStream(st);
  ShutdownTensorEngine<gpu>();
  return rc;
}

}  // namespace

extern "C" int msb_api_suite_run(int id, const float *a, const float *b, float *out, int rows, int cols) {
  try {
    return RunCase(id, a, b, out, rows, cols);
  } catch (const dmlc::Error &e) {
    fprintf(stderr, "api_suite case %d: %s\n", id, e.what());
    return -2;
  }
}
extern "C" int msb_api_suite_num_cases(void) { return 16; }
