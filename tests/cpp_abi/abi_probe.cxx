// Compiled against the REFERENCE's own public headers (not this repository's) and linked against the drop-in:
// virtual-call slots, the header-inline ptr<T>() accessor (shadow pointers), de::Number and de::DH must line up.
#include <cstdint>
#include "DECX/classes/Matrix.h"
#include "DECX/classes/GPU_Matrix.h"
#include "DECX/classes/DecxNumber.h"
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
    std::printf(bad ? "ABI MISMATCH\n" : "abi probe ok\n");
    return bad;
}
