// Scalar arithmetic for the four Standard-algebra element types
// (tenferro-algebra/src/lib.rs:58-72): float, double, float2 (Complex32), double2 (Complex64).
#pragma once
#include <cfloat>

#include "common.h"

namespace tfb {

template <typename T>
struct Ops;

template <>
struct Ops<float> {
    using Real = float;
    static constexpr bool is_complex = false;
    __host__ __device__ static float zero() { return 0.f; }
    __host__ __device__ static float from(Scalar s) { return (float)s.re; }
    __device__ static float add(float a, float b) { return a + b; }
    __device__ static float mul(float a, float b) { return a * b; }
    __device__ static float fma_(float a, float b, float c) { return fmaf(a, b, c); }
    __device__ static float conj(float a) { return a; }
    __device__ static float lowest() { return -INFINITY; }
    __device__ static float highest() { return INFINITY; }
    __device__ static float max_(float a, float b) { return a != a ? a : (b != b ? b : (a > b ? a : b)); }
    __device__ static float min_(float a, float b) { return a != a ? a : (b != b ? b : (a < b ? a : b)); }
    __device__ static float shfl_down(float a, int s) { return __shfl_down_sync(0xffffffffu, a, s); }
};

template <>
struct Ops<double> {
    using Real = double;
    static constexpr bool is_complex = false;
    __host__ __device__ static double zero() { return 0.0; }
    __host__ __device__ static double from(Scalar s) { return s.re; }
    __device__ static double add(double a, double b) { return a + b; }
    __device__ static double mul(double a, double b) { return a * b; }
    __device__ static double fma_(double a, double b, double c) { return fma(a, b, c); }
    __device__ static double conj(double a) { return a; }
    __device__ static double lowest() { return -INFINITY; }
    __device__ static double highest() { return INFINITY; }
    __device__ static double max_(double a, double b) { return a != a ? a : (b != b ? b : (a > b ? a : b)); }
    __device__ static double min_(double a, double b) { return a != a ? a : (b != b ? b : (a < b ? a : b)); }
    __device__ static double shfl_down(double a, int s) { return __shfl_down_sync(0xffffffffu, a, s); }
};

template <>
struct Ops<float2> {
    using Real = float;
    static constexpr bool is_complex = true;
    __host__ __device__ static float2 zero() { return make_float2(0.f, 0.f); }
    __host__ __device__ static float2 from(Scalar s) { return make_float2((float)s.re, (float)s.im); }
    __device__ static float2 add(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
    __device__ static float2 mul(float2 a, float2 b) {
        return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
    }
    __device__ static float2 fma_(float2 a, float2 b, float2 c) {
        c.x = fmaf(a.x, b.x, c.x);
        c.x = fmaf(-a.y, b.y, c.x);
        c.y = fmaf(a.x, b.y, c.y);
        c.y = fmaf(a.y, b.x, c.y);
        return c;
    }
    __device__ static float2 conj(float2 a) { return make_float2(a.x, -a.y); }
    __device__ static float2 lowest() { return zero(); }
    __device__ static float2 highest() { return zero(); }
    __device__ static float2 max_(float2 a, float2) { return a; }
    __device__ static float2 min_(float2 a, float2) { return a; }
    __device__ static float2 shfl_down(float2 a, int s) {
        return make_float2(__shfl_down_sync(0xffffffffu, a.x, s), __shfl_down_sync(0xffffffffu, a.y, s));
    }
};

template <>
struct Ops<double2> {
    using Real = double;
    static constexpr bool is_complex = true;
    __host__ __device__ static double2 zero() { return make_double2(0.0, 0.0); }
    __host__ __device__ static double2 from(Scalar s) { return make_double2(s.re, s.im); }
    __device__ static double2 add(double2 a, double2 b) { return make_double2(a.x + b.x, a.y + b.y); }
    __device__ static double2 mul(double2 a, double2 b) {
        return make_double2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
    }
    __device__ static double2 fma_(double2 a, double2 b, double2 c) {
        c.x = fma(a.x, b.x, c.x);
        c.x = fma(-a.y, b.y, c.x);
        c.y = fma(a.x, b.y, c.y);
        c.y = fma(a.y, b.x, c.y);
        return c;
    }
    __device__ static double2 conj(double2 a) { return make_double2(a.x, -a.y); }
    __device__ static double2 lowest() { return zero(); }
    __device__ static double2 highest() { return zero(); }
    __device__ static double2 max_(double2 a, double2) { return a; }
    __device__ static double2 min_(double2 a, double2) { return a; }
    __device__ static double2 shfl_down(double2 a, int s) {
        return make_double2(__shfl_down_sync(0xffffffffu, a.x, s), __shfl_down_sync(0xffffffffu, a.y, s));
    }
};

// Semirings (tenferro-algebra/src/lib.rs:74-106: zero, one, add, mul).  ALG 0 is the Standard
// algebra (+, *) of all four element types; ALG 1 is MaxPlus (add = max, mul = +, zero = -inf,
// one = 0) and ALG 2 MinPlus (add = min, zero = +inf), both for the real types.  `fma_(a, b, c)`
// is c (+) a (x) b, the step of a contraction's inner loop.
template <typename T, int ALG>
struct Semi {
    __device__ static T zero() { return Ops<T>::zero(); }
    __device__ static T add(T a, T b) { return Ops<T>::add(a, b); }
    __device__ static T mul(T a, T b) { return Ops<T>::mul(a, b); }
    __device__ static T fma_(T a, T b, T c) { return Ops<T>::fma_(a, b, c); }
};
template <typename T>
struct Semi<T, 1> {
    __device__ static T zero() { return Ops<T>::lowest(); }
    __device__ static T add(T a, T b) { return Ops<T>::max_(a, b); }
    __device__ static T mul(T a, T b) { return a + b; }
    __device__ static T fma_(T a, T b, T c) { return Ops<T>::max_(c, a + b); }
};
template <typename T>
struct Semi<T, 2> {
    __device__ static T zero() { return Ops<T>::highest(); }
    __device__ static T add(T a, T b) { return Ops<T>::min_(a, b); }
    __device__ static T mul(T a, T b) { return a + b; }
    __device__ static T fma_(T a, T b, T c) { return Ops<T>::min_(c, a + b); }
};

// V elements moved as one access.
template <typename T, int V>
struct __align__(sizeof(T) * V) Pack {
    T v[V];
};

// out = alpha * (conj?)v + beta * out.  `plain` (alpha = 1, beta = 0, no conj) moves the bits
// untouched, which is what makes Permute bit-exact; beta = 0 never reads the output.
template <typename T>
struct EpilogueArgs {
    T alpha, beta;
    bool plain, read_out, conj, alpha_one;
    static EpilogueArgs make(Scalar a, Scalar b, bool cj) {
        EpilogueArgs e;
        e.alpha = Ops<T>::from(a);
        e.beta = Ops<T>::from(b);
        e.conj = cj && Ops<T>::is_complex;
        e.read_out = !b.is_zero();
        e.alpha_one = a.is_one();
        e.plain = e.alpha_one && !e.read_out && !e.conj;
        return e;
    }
    __device__ __forceinline__ T apply(T v, const T* out) const {
        if (plain) return v;
        if (conj) v = Ops<T>::conj(v);
        if (!alpha_one) v = Ops<T>::mul(alpha, v);
        if (read_out) v = Ops<T>::add(v, Ops<T>::mul(beta, *out));
        return v;
    }
};

}  // namespace tfb
