// Compiled against the REFERENCE's own public headers (not this repository's) and linked against the drop-in:
// virtual-call slots, the header-inline ptr<T>() accessor (shadow pointers), de::Number and de::DH must line up.
#include <cstdint>
#include "DECX/classes/Matrix.h"
#include "DECX/classes/GPU_Matrix.h"
#include "DECX/classes/DecxNumber.h"
#include "DECX/classes/Tensor.h"
#include "DECX/classes/TensorArray.h"
#include "DECX/classes/GPU_Tensor.h"
#include "DECX/classes/GPU_TensorArray.h"
#include <cstdio>
int main() {
    de::Matrix& m = de::CreateMatrixRef(de::_FP32_, 13, 7);
    int bad = 0;
    bad += !(m.Width() == 13 && m.Height() == 7 && m.Type() == de::_FP32_ && m.Format() == de::_NA_);
    *m.ptr<float>(6, 12) = 5.f;
    bad += !(m.ptr<float>(1, 0) - m.ptr<float>(0, 0) == 16);
    de::Matrix& s = de::CreateMatrixRef();
    s.SoftCopy(m);
    bad += !(*s.ptr<float>(6, 12) == 5.f);
    m.Reinterpret(de::_INT32_);
    bad += !(m.Type() == de::_INT32_);
    m.release();
    de::Number n(2.5f);
    bad += !(sizeof(de::Number) == 32 && n.Type() == de::_FP32_ && sizeof(de::DH) == 104);
    // tensors: slots, the two shadow members behind ptr<T>(), the layout record they point to
    de::Tensor& t = de::CreateTensorRef(de::_FP32_, 13, 7, 3);
    bad += !(t.Width() == 13 && t.Height() == 7 && t.Depth() == 3 && t.Type() == de::_FP32_);
    *t.ptr<float>(6, 12, 2) = 4.f;
    bad += !(t.ptr<float>(0, 1, 0) - t.ptr<float>(0, 0, 0) == 4 && t.ptr<float>(1, 0, 0) - t.ptr<float>(0, 0, 0) == 64);
    de::Tensor& t2 = de::CreateTensorRef();
    t2.SoftCopy(t);
    t.release();
    bad += !(*t2.ptr<float>(6, 12, 2) == 4.f);
    de::TensorArray& a = de::CreateTensorArrayRef(de::_FP32_, 5, 3, 6, 4);
    bad += !(a.Width() == 5 && a.Height() == 3 && a.Depth() == 6 && a.TensorNum() == 4 && a.Type() == de::_FP32_);
    *a.ptr<float>(2, 4, 5, 3) = 9.f;
    de::Tensor& sl = de::CreateTensorRef();
    bad += !(a.Extract_SoftCopy(3, sl).error_type == 0 && *sl.ptr<float>(2, 4, 5) == 9.f);
    a.release();
    bad += !(*sl.ptr<float>(2, 4, 5) == 9.f);
    sl.release();
    t2.release();
    de::GPU_Tensor& g = de::CreateGPUTensorRef();            // empty objects: no device is touched
    de::GPU_TensorArray& ga = de::CreateGPUTensorArrayRef();
    bad += !(g.Width() == 0 && g.Depth() == 0 && ga.TensorNum() == 0 && ga.Height() == 0);
    g.release();
    ga.release();
    std::printf(bad ? "ABI MISMATCH\n" : "abi probe ok\n");
    return bad;
}
