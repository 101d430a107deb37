// Math vocabulary of generated bodies: one function per Inductor op, overloaded for
// scalar and per-thread-vector operands (gen_vec.cuh).  Floating values are always fp32
// (half inputs are widened on load, inductor_x/codegen/triton.py:1431-1433), integers are
// 64-bit, booleans are bool.
#pragma once
#include "gen_vec.cuh"

namespace ixb {
namespace gen {
namespace op {

#define IXB_OP_F1(NAME, EXPR)                                                       \
  template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type NAME(const A& a) { \
    return map1<typename fres<rank<A>::n>::type>([](float x) { return (EXPR); }, a);  \
  }
// exp / sigmoid use the hardware exponential (ex2.approx on a pre-scaled argument), as
// Inductor's GPU code generation does for these ops
IXB_OP_F1(exp, __expf(x))
IXB_OP_F1(exp2, exp2f(x))
IXB_OP_F1(expm1, expm1f(x))
IXB_OP_F1(log, logf(x))
IXB_OP_F1(log2, log2f(x))
IXB_OP_F1(log10, log10f(x))
IXB_OP_F1(log1p, log1pf(x))
IXB_OP_F1(sqrt, sqrtf(x))
IXB_OP_F1(rsqrt, rsqrtf(x))
IXB_OP_F1(sin, sinf(x))
IXB_OP_F1(cos, cosf(x))
IXB_OP_F1(tan, tanf(x))
IXB_OP_F1(asin, asinf(x))
IXB_OP_F1(acos, acosf(x))
IXB_OP_F1(atan, atanf(x))
IXB_OP_F1(sinh, sinhf(x))
IXB_OP_F1(cosh, coshf(x))
IXB_OP_F1(tanh, tanhf(x))
IXB_OP_F1(erf, erff(x))
IXB_OP_F1(erfc, erfcf(x))
IXB_OP_F1(lgamma, lgammaf(x))
IXB_OP_F1(floor, floorf(x))
IXB_OP_F1(ceil, ceilf(x))
IXB_OP_F1(trunc, truncf(x))
IXB_OP_F1(round, nearbyintf(x))
IXB_OP_F1(reciprocal, 1.f / x)
IXB_OP_F1(sigmoid, __fdividef(1.f, 1.f + __expf(-x)))
IXB_OP_F1(to_float, x)
#undef IXB_OP_F1

// abs / neg / square / relu / sign keep the operand's kind (int stays int)
#define IXB_OP_SAME1(NAME, FEXPR, IEXPR)                                                        \
  template <class A> __device__ __forceinline__ auto NAME(const A& a) {                         \
    if constexpr (is_intlike<A>::value) {                                                       \
      return map1<typename ires<rank<A>::n>::type>([](long long x) { return (long long)(IEXPR); }, a); \
    } else {                                                                                    \
      return map1<typename fres<rank<A>::n>::type>([](float x) { return (float)(FEXPR); }, a);  \
    }                                                                                           \
  }
IXB_OP_SAME1(abs, fabsf(x), (x < 0 ? -x : x))
IXB_OP_SAME1(neg, -x, -x)
IXB_OP_SAME1(square, x * x, x * x)
IXB_OP_SAME1(relu, (x != x ? x : fmaxf(x, 0.f)), (x > 0 ? x : 0))
IXB_OP_SAME1(sign, ((x > 0.f) - (x < 0.f)), ((x > 0) - (x < 0)))
#undef IXB_OP_SAME1

template <class A> __device__ __forceinline__ typename bres<rank<A>::n>::type isnan(const A& a) {
  return map1<typename bres<rank<A>::n>::type>([](float x) { return x != x; }, a);
}
template <class A> __device__ __forceinline__ typename bres<rank<A>::n>::type isinf(const A& a) {
  return map1<typename bres<rank<A>::n>::type>([](float x) { return ::isinf(x) != 0; }, a);
}
template <class A> __device__ __forceinline__ typename bres<rank<A>::n>::type signbit(const A& a) {
  return map1<typename bres<rank<A>::n>::type>([](float x) { return ::signbit(x) != 0; }, a);
}
template <class A> __device__ __forceinline__ typename ires<rank<A>::n>::type to_int(const A& a) {
  if constexpr (is_intlike<A>::value || is_boollike<A>::value) {
    return map1<typename ires<rank<A>::n>::type>([](long long x) { return x; }, a);
  } else {
    return map1<typename ires<rank<A>::n>::type>([](float x) { return (long long)x; }, a);
  }
}
template <class A> __device__ __forceinline__ typename bres<rank<A>::n>::type to_bool(const A& a) {
  if constexpr (is_intlike<A>::value || is_boollike<A>::value) {
    return map1<typename bres<rank<A>::n>::type>([](long long x) { return x != 0; }, a);
  } else {
    return map1<typename bres<rank<A>::n>::type>([](float x) { return x != 0.f; }, a);
  }
}
// value as it would read after a round trip through a 16-bit storage type
template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type round_bf16(const A& a) {
  return map1<typename fres<rank<A>::n>::type>(
      [](float x) { return __bfloat162float(__float2bfloat16_rn(x)); }, a);
}
template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type round_f16(const A& a) {
  return map1<typename fres<rank<A>::n>::type>([](float x) { return __half2float(__float2half_rn(x)); },
                                               a);
}

// ---- binary ---------------------------------------------------------------------------
#define IXB_OP_F2(NAME, EXPR)                                                                  \
  template <class A, class B>                                                                  \
  __device__ __forceinline__ typename fres<rank2<A, B>::n>::type NAME(const A& a, const B& b) { \
    return map2<typename fres<rank2<A, B>::n>::type>([](float x, float y) { return (EXPR); }, a, b); \
  }
// division by a value that does not vary along the vector (a row statistic) is one
// reciprocal and N multiplies
template <class A, class B>
__device__ __forceinline__ typename fres<rank2<A, B>::n>::type truediv(const A& a, const B& b) {
  if constexpr (rank<B>::n == 0 && rank<A>::n > 0) {
    const float inv = 1.f / (float)at(b, 0);
    return map1<typename fres<rank<A>::n>::type>([inv](float x) { return x * inv; }, a);
  } else {
    return map2<typename fres<rank2<A, B>::n>::type>([](float x, float y) { return x / y; }, a, b);
  }
}
IXB_OP_F2(pow, powf(x, y))
IXB_OP_F2(fmod, fmodf(x, y))
IXB_OP_F2(atan2, atan2f(x, y))
IXB_OP_F2(copysign, copysignf(x, y))
IXB_OP_F2(hypot, hypotf(x, y))
#undef IXB_OP_F2

// kind-preserving binary ops (int with int stays int); max/min propagate NaN like torch
#define IXB_OP_ARITH2(NAME, FEXPR, IEXPR)                                                      \
  template <class A, class B>                                                                  \
  __device__ __forceinline__ typename arith<A, B>::type NAME(const A& a, const B& b) {         \
    if constexpr (arith<A, B>::ints) {                                                         \
      return map2<typename arith<A, B>::type>(                                                 \
          [](long long x, long long y) { return (long long)(IEXPR); }, a, b);                  \
    } else {                                                                                   \
      return map2<typename arith<A, B>::type>([](float x, float y) { return (float)(FEXPR); }, a, b); \
    }                                                                                          \
  }
IXB_OP_ARITH2(add, x + y, x + y)
IXB_OP_ARITH2(sub, x - y, x - y)
IXB_OP_ARITH2(mul, x * y, x * y)
IXB_OP_ARITH2(maximum, (x != x ? x : (y != y ? y : fmaxf(x, y))), (x > y ? x : y))
IXB_OP_ARITH2(minimum, (x != x ? x : (y != y ? y : fminf(x, y))), (x < y ? x : y))
// python-style floor division and modulo for integers, C-style truncation for truncdiv
IXB_OP_ARITH2(floordiv, floorf(x / y), ((x / y) - ((x % y != 0) && ((x < 0) != (y < 0)))))
IXB_OP_ARITH2(truncdiv, truncf(x / y), x / y)
IXB_OP_ARITH2(remainder, (x - y * floorf(x / y)), ((x % y) + (((x % y) != 0 && ((x % y) < 0) != (y < 0)) ? y : 0)))
IXB_OP_ARITH2(mod, fmodf(x, y), x % y)
#undef IXB_OP_ARITH2

// index arithmetic: operands are non-negative, so C truncation equals floor
template <class A, class B>
__device__ __forceinline__ typename ires<rank2<A, B>::n>::type idiv(const A& a, const B& b) {
  return map2<typename ires<rank2<A, B>::n>::type>([](long long x, long long y) { return x / y; }, a, b);
}
template <class A, class B>
__device__ __forceinline__ typename ires<rank2<A, B>::n>::type imod(const A& a, const B& b) {
  return map2<typename ires<rank2<A, B>::n>::type>([](long long x, long long y) { return x % y; }, a, b);
}

#define IXB_OP_B2(NAME, EXPR)                                                                  \
  template <class A, class B>                                                                  \
  __device__ __forceinline__ typename bres<rank2<A, B>::n>::type NAME(const A& a, const B& b) { \
    return map2<typename bres<rank2<A, B>::n>::type>([](bool x, bool y) { return (EXPR); }, a, b); \
  }
IXB_OP_B2(logical_and, x && y)
IXB_OP_B2(logical_or, x || y)
IXB_OP_B2(logical_xor, x != y)
#undef IXB_OP_B2
template <class A> __device__ __forceinline__ typename bres<rank<A>::n>::type logical_not(const A& a) {
  return map1<typename bres<rank<A>::n>::type>([](bool x) { return !x; }, a);
}

#define IXB_OP_CMP(NAME, OP)                                                                   \
  template <class A, class B>                                                                  \
  __device__ __forceinline__ typename bres<rank2<A, B>::n>::type NAME(const A& a, const B& b) { \
    using E = typename arith<A, B>::elem;                                                      \
    return map2<typename bres<rank2<A, B>::n>::type>([](E x, E y) { return x OP y; }, a, b);   \
  }
IXB_OP_CMP(eq, ==)
IXB_OP_CMP(ne, !=)
IXB_OP_CMP(lt, <)
IXB_OP_CMP(le, <=)
IXB_OP_CMP(gt, >)
IXB_OP_CMP(ge, >=)
#undef IXB_OP_CMP

// where(c, a, b): result kind follows a / b
template <class C, class A, class B>
__device__ __forceinline__ auto where(const C& c, const A& a, const B& b) {
  constexpr int N = rank3<C, A, B>::n;
  if constexpr (is_boollike<A>::value && is_boollike<B>::value) {
    return map3<typename bres<N>::type>([](bool m, bool x, bool y) { return m ? x : y; }, c, a, b);
  } else if constexpr (arith<A, B>::ints) {
    return map3<typename ires<N>::type>([](bool m, long long x, long long y) { return m ? x : y; }, c, a, b);
  } else {
    return map3<typename fres<N>::type>([](bool m, float x, float y) { return m ? x : y; }, c, a, b);
  }
}

}  // namespace op
}  // namespace gen
}  // namespace ixb
