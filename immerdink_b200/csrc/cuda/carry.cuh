// Multiword subtract with borrow on 32-bit words as single PTX carry chains (one instruction per
// word). d = a - b; returns 1 when a < b (the result is then the two's complement of b - a).
#pragma once
#include <cstdint>

namespace imd {
namespace dev {

template <int W>
struct Words;

template <>
struct Words<1> {
  static __device__ __forceinline__ uint32_t sub(uint32_t* d, const uint32_t* a, const uint32_t* b) {
    uint32_t br;
    asm("sub.cc.u32 %0, %2, %3;\n\tsubc.u32 %1, 0, 0;"
        : "=r"(d[0]), "=r"(br) : "r"(a[0]), "r"(b[0]));
    return br & 1u;
  }
};
template <>
struct Words<2> {
  static __device__ __forceinline__ uint32_t sub(uint32_t* d, const uint32_t* a, const uint32_t* b) {
    uint32_t br;
    asm("sub.cc.u32 %0, %3, %5;\n\tsubc.cc.u32 %1, %4, %6;\n\tsubc.u32 %2, 0, 0;"
        : "=r"(d[0]), "=r"(d[1]), "=r"(br) : "r"(a[0]), "r"(a[1]), "r"(b[0]), "r"(b[1]));
    return br & 1u;
  }
};
template <>
struct Words<3> {
  static __device__ __forceinline__ uint32_t sub(uint32_t* d, const uint32_t* a, const uint32_t* b) {
    uint32_t br;
    asm("sub.cc.u32 %0, %4, %7;\n\tsubc.cc.u32 %1, %5, %8;\n\tsubc.cc.u32 %2, %6, %9;\n\t"
        "subc.u32 %3, 0, 0;"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(br)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(b[0]), "r"(b[1]), "r"(b[2]));
    return br & 1u;
  }
};
template <>
struct Words<4> {
  static __device__ __forceinline__ uint32_t sub(uint32_t* d, const uint32_t* a, const uint32_t* b) {
    uint32_t br;
    asm("sub.cc.u32 %0, %5, %9;\n\tsubc.cc.u32 %1, %6, %10;\n\tsubc.cc.u32 %2, %7, %11;\n\t"
        "subc.cc.u32 %3, %8, %12;\n\tsubc.u32 %4, 0, 0;"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(br)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(b[2]), "r"(b[3]));
    return br & 1u;
  }
};
template <>
struct Words<5> {
  static __device__ __forceinline__ uint32_t sub(uint32_t* d, const uint32_t* a, const uint32_t* b) {
    uint32_t br;
    asm("sub.cc.u32 %0, %6, %11;\n\tsubc.cc.u32 %1, %7, %12;\n\tsubc.cc.u32 %2, %8, %13;\n\t"
        "subc.cc.u32 %3, %9, %14;\n\tsubc.cc.u32 %4, %10, %15;\n\tsubc.u32 %5, 0, 0;"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(br)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(b[0]), "r"(b[1]), "r"(b[2]),
          "r"(b[3]), "r"(b[4]));
    return br & 1u;
  }
};
template <>
struct Words<6> {
  static __device__ __forceinline__ uint32_t sub(uint32_t* d, const uint32_t* a, const uint32_t* b) {
    uint32_t br;
    asm("sub.cc.u32 %0, %7, %13;\n\tsubc.cc.u32 %1, %8, %14;\n\tsubc.cc.u32 %2, %9, %15;\n\t"
        "subc.cc.u32 %3, %10, %16;\n\tsubc.cc.u32 %4, %11, %17;\n\tsubc.cc.u32 %5, %12, %18;\n\t"
        "subc.u32 %6, 0, 0;"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]), "=r"(d[4]), "=r"(d[5]), "=r"(br)
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(a[4]), "r"(a[5]), "r"(b[0]), "r"(b[1]),
          "r"(b[2]), "r"(b[3]), "r"(b[4]), "r"(b[5]));
    return br & 1u;
  }
};

}  // namespace dev
}  // namespace imd
