// Small value types used by the GEMM path (reference: srcs/includes/DECX/classes/class_utils.h:19-75).
#ifndef DECX_B200_PUBLIC_CLASS_UTILS_H_
#define DECX_B200_PUBLIC_CLASS_UTILS_H_

#include "../basic.h"
#include "type_info.h"

namespace de {

struct Half {
    unsigned short val;   // IEEE binary16 bits
};

typedef struct __align__(8) complex_f {
    float real, image;
    complex_f(const float re, const float im) : real(re), image(im) {}
    complex_f() {}
} CPf;

typedef struct __align__(16) complex_d {
    double real, image;
    complex_d(const double re, const double im) : real(re), image(im) {}
    complex_d() : real(0), image(0) {}
} CPd;

// {x = column, y = row} wherever a Point2D addresses a matrix
struct __align__(8) Point2D {
    int32_t x, y;
    Point2D(const int32_t _x, const int32_t _y) : x(_x), y(_y) {}
    Point2D(const uint32_t _x, const uint32_t _y) : x(int32_t(_x)), y(int32_t(_y)) {}
    Point2D() {}
};

// {x = depth (channel), y = column, z = row} wherever a Point3D addresses a tensor
struct __align__(16) Point3D {
    int32_t x, y, z;
    Point3D(const int32_t _x, const int32_t _y, const int32_t _z) : x(_x), y(_y), z(_z) {}
    Point3D(const uint32_t _x, const uint32_t _y, const uint32_t _z) : x(int32_t(_x)), y(int32_t(_y)), z(int32_t(_z)) {}
    Point3D() {}
};

}  // namespace de
#endif
