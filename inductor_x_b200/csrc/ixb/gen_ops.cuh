// Math vocabulary of generated bodies: one function per Inductor op, overloaded for
// scalar and per-thread-vector operands (gen_vec.cuh).  Floating values are always fp32
// (half inputs are widened on load, inductor_x/codegen/triton.py:1431-1433), integers are
// 64-bit, booleans are bool.
#pragma once
#include "gen_vec.cuh"

namespace ixb {
namespace gen {
namespace op {

// ---- packed fp32 pairs ----------------------------------------------------------------
// sm_100 issues fma/mul/add on two fp32 lanes per instruction (f32x2).  Whenever an
// arithmetic op produces a float vector of even length from float vectors and float
// scalars, it runs pair by pair through those instructions: half the issue slots of the
// scalar form.  Integer or boolean operands take the element-wise path.
template <class T> struct is_fvec { static constexpr bool value = false; };
template <int N> struct is_fvec<vf<N>> { static constexpr bool value = (N % 2) == 0; };
template <class T> struct is_fany { static constexpr bool value = is_fvec<T>::value || std::is_same<T, float>::value; };
template <class A, class B> struct packable2 {
  static constexpr bool value = (is_fvec<A>::value || is_fvec<B>::value) && is_fany<A>::value && is_fany<B>::value;
};
template <class A, class B, class C> struct packable3 {
  static constexpr bool value = (is_fvec<A>::value || is_fvec<B>::value || is_fvec<C>::value) &&
                                is_fany<A>::value && is_fany<B>::value && is_fany<C>::value;
};
template <int N> __device__ __forceinline__ float2 pr(const vf<N>& a, int p) { return make_float2(a.v[2 * p], a.v[2 * p + 1]); }
__device__ __forceinline__ float2 pr(float a, int) { return make_float2(a, a); }
template <int N> __device__ __forceinline__ void set_pr(vf<N>& r, int p, float2 d) {
  r.v[2 * p] = d.x;
  r.v[2 * p + 1] = d.y;
}

// a * b + c with a single rounding (what the compiler's contraction of a*b+c gives for
// scalar code; the emitter contracts explicitly because packed instructions are opaque to it)
template <class A, class B, class C>
__device__ __forceinline__ typename fres<rank3<A, B, C>::n>::type fma(const A& a, const B& b, const C& c) {
  constexpr int N = rank3<A, B, C>::n;
  if constexpr (packable3<A, B, C>::value) {
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) set_pr(r, p, fma2(pr(a, p), pr(b, p), pr(c, p)));
    return r;
  } else {
    return map3<typename fres<N>::type>([](float x, float y, float z) { return fmaf(x, y, z); }, a, b, c);
  }
}

#define IXB_OP_F1(NAME, EXPR)                                                       \
  template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type NAME(const A& a) { \
    return map1<typename fres<rank<A>::n>::type>([](float x) { return (EXPR); }, a);  \
  }
// exp / sigmoid use the hardware exponential (ex2.approx on a pre-scaled argument), as
// Inductor's GPU code generation does for these ops
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
IXB_OP_F1(erfc, erfcf(x))
IXB_OP_F1(asinh, asinhf(x))
IXB_OP_F1(acosh, acoshf(x))
IXB_OP_F1(atanh, atanhf(x))
IXB_OP_F1(erfinv, erfinvf(x))
IXB_OP_F1(lgamma, lgammaf(x))
IXB_OP_F1(floor, floorf(x))
IXB_OP_F1(ceil, ceilf(x))
IXB_OP_F1(trunc, truncf(x))
IXB_OP_F1(round, nearbyintf(x))
IXB_OP_F1(reciprocal, 1.f / x)
IXB_OP_F1(to_float, x)
#undef IXB_OP_F1

// exp(x) = 2^(x * log2 e) on the hardware exponential (ex2.approx), as Inductor's GPU code
// generation does; the pre-scale runs on packed pairs
template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type exp(const A& a) {
  if constexpr (is_fvec<A>::value) {
    constexpr int N = rank<A>::n;
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) {
      const float2 t = mul2(pr(a, p), make_float2(kLog2e, kLog2e));
      set_pr(r, p, make_float2(fast_exp2(t.x), fast_exp2(t.y)));
    }
    return r;
  } else {
    return map1<typename fres<rank<A>::n>::type>([](float x) { return fast_exp2(x * kLog2e); }, a);
  }
}
// exp(a - b) where b does not vary along the vector (a row statistic): the subtraction and
// the pre-scale are one packed fma, 2^(a * log2 e - b * log2 e).  The product b * log2 e
// is rounded once more than in exp(a - b); the emitter uses this form for groups stored in
// 16-bit types only.
template <class A>
__device__ __forceinline__ typename fres<rank<A>::n>::type exp_sub(const A& a, float b) {
  const float nb = -b * kLog2e;
  if constexpr (is_fvec<A>::value) {
    constexpr int N = rank<A>::n;
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) {
      const float2 t = fma2(pr(a, p), make_float2(kLog2e, kLog2e), make_float2(nb, nb));
      set_pr(r, p, make_float2(fast_exp2(t.x), fast_exp2(t.y)));
    }
    return r;
  } else {
    return map1<typename fres<rank<A>::n>::type>([nb](float x) { return fast_exp2(fmaf(x, kLog2e, nb)); }, a);
  }
}
template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type sigmoid(const A& a) {
  if constexpr (is_fvec<A>::value) {
    constexpr int N = rank<A>::n;
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) {
      const float2 t = mul2(pr(a, p), make_float2(-kLog2e, -kLog2e));
      const float2 d = add2(make_float2(fast_exp2(t.x), fast_exp2(t.y)), make_float2(1.f, 1.f));
      set_pr(r, p, make_float2(__fdividef(1.f, d.x), __fdividef(1.f, d.y)));
    }
    return r;
  } else {
    return map1<typename fres<rank<A>::n>::type>(
        [](float x) { return __fdividef(1.f, 1.f + fast_exp2(-x * kLog2e)); }, a);
  }
}

// erf on two values at once, branch-free: |x| <= 1 takes x * P(x^2) (degree 5, relative
// error 4e-8 against the fp64 function), larger arguments take 1 - 2^-Q(|x|) with Q a
// degree-6 fit of -log2(erfc) on [1, 4] (absolute error 1e-9); beyond 4 the result is +-1.
// Both branches run on packed pairs and a select picks per element.
__device__ __forceinline__ float2 erf2(float2 x) {
  const float2 t = make_float2(fminf(fabsf(x.x), 4.f), fminf(fabsf(x.y), 4.f));
  const float2 s = mul2(x, x);
#define IXB_C2(v) make_float2(v, v)
  float2 p = fma2(IXB_C2(-0.0005631402018480003f), s, IXB_C2(0.004917546175420284f));
  p = fma2(p, s, IXB_C2(-0.02671130746603012f));
  p = fma2(p, s, IXB_C2(0.11280179768800735f));
  p = fma2(p, s, IXB_C2(-0.37612324953079224f));
  p = fma2(p, s, IXB_C2(1.1283791065216064f));
  p = mul2(p, x);
  // coefficients negated: the polynomial yields -Q, the argument of the exponential
  float2 q = fma2(IXB_C2(0.0002677357697393745f), t, IXB_C2(-0.004241043236106634f));
  q = fma2(q, t, IXB_C2(0.03145876154303551f));
  q = fma2(q, t, IXB_C2(-0.14865218102931976f));
  q = fma2(q, t, IXB_C2(-0.9207642674446106f));
  q = fma2(q, t, IXB_C2(-1.625975489616394f));
  q = fma2(q, t, IXB_C2(-0.0005102010909467936f));
#undef IXB_C2
  const float bx = copysignf(1.f - fast_exp2(q.x), x.x);
  const float by = copysignf(1.f - fast_exp2(q.y), x.y);
  return make_float2(fabsf(x.x) > 1.f ? bx : p.x, fabsf(x.y) > 1.f ? by : p.y);
}
template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type erf(const A& a) {
  if constexpr (is_fvec<A>::value) {
    constexpr int N = rank<A>::n;
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) set_pr(r, p, erf2(pr(a, p)));
    return r;
  } else {
    return map1<typename fres<rank<A>::n>::type>([](float x) { return erf2(make_float2(x, x)).x; }, a);
  }
}
// exact-erf GELU, 0.5 * v * (1 + erf(v / sqrt 2)), through the fitted form of common.cuh
// (absolute error 2.8e-7): the emitter prints this when it recognises the decomposed graph
template <class A> __device__ __forceinline__ typename fres<rank<A>::n>::type gelu_erf(const A& a) {
  if constexpr (is_fvec<A>::value) {
    constexpr int N = rank<A>::n;
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) set_pr(r, p, gelu_erf_fast2(pr(a, p)));
    return r;
  } else {
    return map1<typename fres<rank<A>::n>::type>([](float x) { return gelu_erf_fast(x); }, a);
  }
}

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
  if constexpr (rank<B>::n == 0 && is_fvec<A>::value) {
    const float inv = 1.f / (float)at(b, 0);
    constexpr int N = rank<A>::n;
    vf<N> r;
#pragma unroll
    for (int p = 0; p < N / 2; ++p) set_pr(r, p, mul2(pr(a, p), make_float2(inv, inv)));
    return r;
  } else if constexpr (rank<B>::n == 0 && rank<A>::n > 0) {
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
IXB_OP_F2(nextafter, nextafterf(x, y))
IXB_OP_F2(ldexp, ldexpf(x, (int)y))
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
#define IXB_OP_PACKED2(NAME, PEXPR, FEXPR, IEXPR)                                               \
  template <class A, class B>                                                                  \
  __device__ __forceinline__ typename arith<A, B>::type NAME(const A& a, const B& b) {         \
    if constexpr (packable2<A, B>::value) {                                                    \
      constexpr int N = rank2<A, B>::n;                                                        \
      vf<N> r;                                                                                 \
      _Pragma("unroll") for (int p = 0; p < N / 2; ++p) {                                      \
        const float2 x = pr(a, p), y = pr(b, p);                                               \
        set_pr(r, p, (PEXPR));                                                                 \
      }                                                                                        \
      return r;                                                                                \
    } else if constexpr (arith<A, B>::ints) {                                                  \
      return map2<typename arith<A, B>::type>(                                                 \
          [](long long x, long long y) { return (long long)(IEXPR); }, a, b);                  \
    } else {                                                                                   \
      return map2<typename arith<A, B>::type>([](float x, float y) { return (float)(FEXPR); }, a, b); \
    }                                                                                          \
  }
IXB_OP_PACKED2(add, add2(x, y), x + y, x + y)
IXB_OP_PACKED2(sub, fma2(y, make_float2(-1.f, -1.f), x), x - y, x - y)
IXB_OP_PACKED2(mul, mul2(x, y), x * y, x * y)
#undef IXB_OP_PACKED2
// NaN-propagating like torch.maximum / torch.minimum: one max.NaN / min.NaN instruction
IXB_OP_ARITH2(maximum, MaxOp::combine(x, y), (x > y ? x : y))
IXB_OP_ARITH2(minimum, MinOp::combine(x, y), (x < y ? x : y))
// python-style floor division and modulo for integers, C-style truncation for truncdiv
// floating remainder with the sign of the divisor, from the exact fmod (x - y * floor(x / y)
// would lose every digit once x / y no longer fits the mantissa)
__device__ __forceinline__ float py_fmod(float x, float y) {
  const float r = fmodf(x, y);
  return (r != 0.f && ((r < 0.f) != (y < 0.f))) ? r + y : r;
}
IXB_OP_ARITH2(floordiv, floorf(x / y), ((x / y) - ((x % y != 0) && ((x < 0) != (y < 0)))))
IXB_OP_ARITH2(truncdiv, truncf(x / y), x / y)
IXB_OP_ARITH2(remainder, py_fmod(x, y), ((x % y) + (((x % y) != 0 && ((x % y) < 0) != (y < 0)) ? y : 0)))
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

// bitwise ops of integer operands (booleans take the logical forms above).  Integers are held
// sign-extended (unsigned bytes zero-extended) in 64 bits, so and / or / xor / not of two
// values of one type give that type's result in the same representation; a shift count outside
// [0, 63] gives 0 (left) or the sign fill (right).
#define IXB_OP_I2(NAME, EXPR)                                                                  \
  template <class A, class B>                                                                  \
  __device__ __forceinline__ typename ires<rank2<A, B>::n>::type NAME(const A& a, const B& b) { \
    return map2<typename ires<rank2<A, B>::n>::type>(                                          \
        [](long long x, long long y) { return (long long)(EXPR); }, a, b);                     \
  }
IXB_OP_I2(bit_and, x & y)
IXB_OP_I2(bit_or, x | y)
IXB_OP_I2(bit_xor, x ^ y)
IXB_OP_I2(lshift, ((unsigned long long)y > 63ULL ? 0LL : (long long)((unsigned long long)x << y)))
IXB_OP_I2(rshift, (x >> ((unsigned long long)y > 63ULL ? 63 : y)))
#undef IXB_OP_I2
template <class A> __device__ __forceinline__ typename ires<rank<A>::n>::type bit_not(const A& a) {
  return map1<typename ires<rank<A>::n>::type>([](long long x) { return ~x; }, a);
}
// the value an integer of BITS bits (signed or not) holds after a conversion or an operation
// that can leave its range: two's-complement wrap, back in the 64-bit representation
template <int BITS, bool SIGNED, class A>
__device__ __forceinline__ typename ires<rank<A>::n>::type wrap_int(const A& a) {
  return map1<typename ires<rank<A>::n>::type>(
      [](long long x) {
        if constexpr (BITS == 8 && SIGNED) return (long long)(signed char)x;
        else if constexpr (BITS == 8) return (long long)(unsigned char)x;
        else if constexpr (BITS == 16) return (long long)(short)x;
        else if constexpr (BITS == 32) return (long long)(int)x;
        else return x;
      },
      a);
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
