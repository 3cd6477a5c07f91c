// Elementwise operations with the reference's semantics (emmy_ptx/elementwise.py:1-16,
// tests/oracle.py:10-16): IEEE round-to-nearest float arithmetic that is never contracted when
// EMB_STRICT is set, CUDA's fmaxf/fminf for maximum/minimum (a NaN gives the other operand,
// -0 < +0), numpy's wrap-around and floor division for integers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "emb_math.cuh"

#ifndef EMB_STRICT
#define EMB_STRICT 0
#endif

namespace emb {

#if EMB_STRICT
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double add(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
#else
__device__ __forceinline__ float add(float a, float b) { return a + b; }
__device__ __forceinline__ float sub(float a, float b) { return a - b; }
__device__ __forceinline__ float mul(float a, float b) { return a * b; }
__device__ __forceinline__ double add(double a, double b) { return a + b; }
__device__ __forceinline__ double sub(double a, double b) { return a - b; }
__device__ __forceinline__ double mul(double a, double b) { return a * b; }
#endif
__device__ __forceinline__ float div(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ double div(double a, double b) { return __ddiv_rn(a, b); }
__device__ __forceinline__ float rcp(float a) { return __frcp_rn(a); }
__device__ __forceinline__ double rcp(double a) { return __drcp_rn(a); }
__device__ __forceinline__ float sqrt_(float a) { return __fsqrt_rn(a); }
__device__ __forceinline__ double sqrt_(double a) { return __dsqrt_rn(a); }
__device__ __forceinline__ float maximum(float a, float b) { return fmaxf(a, b); }
__device__ __forceinline__ float minimum(float a, float b) { return fminf(a, b); }
__device__ __forceinline__ double maximum(double a, double b) { return fmax(a, b); }
__device__ __forceinline__ double minimum(double a, double b) { return fmin(a, b); }

// integers: fixed-width two's complement, as numpy arrays compute
template <class T> struct wide { using u = unsigned; };
template <> struct wide<long long> { using u = unsigned long long; };
template <> struct wide<unsigned long long> { using u = unsigned long long; };
#define EMB_INT_OPS(T)                                                                                       \
    __device__ __forceinline__ T add(T a, T b) { return (T)((wide<T>::u)a + (wide<T>::u)b); }                \
    __device__ __forceinline__ T sub(T a, T b) { return (T)((wide<T>::u)a - (wide<T>::u)b); }                \
    __device__ __forceinline__ T mul(T a, T b) { return (T)((wide<T>::u)a * (wide<T>::u)b); }                \
    __device__ __forceinline__ T maximum(T a, T b) { return a > b ? a : b; }                                 \
    __device__ __forceinline__ T minimum(T a, T b) { return a < b ? a : b; }                                 \
    __device__ __forceinline__ T floor_divide(T a, T b) {                                                    \
        if (b == 0) return 0;                                                                                \
        T q = a / b;                                                                                         \
        return (a % b != 0 && ((a % b < 0) != (b < 0))) ? q - 1 : q;                                         \
    }                                                                                                        \
    __device__ __forceinline__ T remainder(T a, T b) {                                                       \
        if (b == 0) return 0;                                                                                \
        T r = a % b;                                                                                         \
        return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r;                                                 \
    }
EMB_INT_OPS(int)
EMB_INT_OPS(unsigned)
EMB_INT_OPS(long long)
EMB_INT_OPS(unsigned long long)
#undef EMB_INT_OPS

// the e4m3 decode (emmy_ptx/elementwise.py:100-110): exact widening through f16
__device__ __forceinline__ float from_f8e4m3(unsigned code) {
    unsigned short pair = static_cast<unsigned short>(code & 0xffu);
    unsigned halves;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(halves) : "h"(pair));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(halves & 0xffffu)));
}

// the other three fp8 conversions of the reference (emmy_ptx/elementwise.py:100-129): e5m2 decoded the same way
// (infinities and NaNs stay); encodes round to nearest even and saturate to the largest finite value, NaN to 0x7f
// (one cvt.rn.satfinite on the pair (x, x), low byte kept)
__device__ __forceinline__ float from_f8e5m2(unsigned code) {
    unsigned short pair = static_cast<unsigned short>(code & 0xffu);
    unsigned halves;
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(halves) : "h"(pair));
    return __half2float(__ushort_as_half(static_cast<unsigned short>(halves & 0xffffu)));
}
__device__ __forceinline__ unsigned char to_f8e4m3(float x) {
    unsigned short pair;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %1;" : "=h"(pair) : "f"(x));
    return static_cast<unsigned char>(pair & 0xffu);
}
__device__ __forceinline__ unsigned char to_f8e5m2(float x) {
    unsigned short pair;
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %1;" : "=h"(pair) : "f"(x));
    return static_cast<unsigned char>(pair & 0xffu);
}

// reduction combines as types, for the templates
struct OpAdd {
    static __device__ __forceinline__ float apply(float a, float b) { return add(a, b); }
    static __device__ __forceinline__ float identity() { return 0.0f; }
};
struct OpMul {
    static __device__ __forceinline__ float apply(float a, float b) { return mul(a, b); }
    static __device__ __forceinline__ float identity() { return 1.0f; }
};
struct OpMax {
    static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
    static __device__ __forceinline__ float identity() { return -1e30f; }
};
struct OpMin {
    static __device__ __forceinline__ float apply(float a, float b) { return fminf(a, b); }
    static __device__ __forceinline__ float identity() { return 1e30f; }
};

}  // namespace emb
