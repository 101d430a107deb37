// Value types and math for generated functor bodies.  A fused node group is emitted as
// straight-line C++ over these types; `vf<N>` / `vi<N>` / `vb<N>` hold the N elements a
// thread owns (fully unrolled, they live in registers) and every operator and function is
// overloaded for scalars and vectors alike, so the emitter prints one expression per op
// regardless of whether its operands vary along the vector.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace ixb {
namespace gen {

template <int N> struct vf { float v[N]; };
template <int N> struct vi { long long v[N]; };
template <int N> struct vb { bool v[N]; };

// scalar "vectors" let one set of templates serve both ranks
template <class T> struct rank { static constexpr int n = 0; };
template <int N> struct rank<vf<N>> { static constexpr int n = N; };
template <int N> struct rank<vi<N>> { static constexpr int n = N; };
template <int N> struct rank<vb<N>> { static constexpr int n = N; };

template <int N> __device__ __forceinline__ float at(const vf<N>& a, int i) { return a.v[i]; }
template <int N> __device__ __forceinline__ long long at(const vi<N>& a, int i) { return a.v[i]; }
template <int N> __device__ __forceinline__ bool at(const vb<N>& a, int i) { return a.v[i]; }
__device__ __forceinline__ float at(float a, int) { return a; }
__device__ __forceinline__ double at(double a, int) { return a; }
__device__ __forceinline__ long long at(long long a, int) { return a; }
__device__ __forceinline__ long long at(long a, int) { return a; }
__device__ __forceinline__ long long at(int a, int) { return a; }
__device__ __forceinline__ bool at(bool a, int) { return a; }

template <class A, class B> struct rank2 {
  static constexpr int n = rank<A>::n > rank<B>::n ? rank<A>::n : rank<B>::n;
};
template <class A, class B, class C> struct rank3 {
  static constexpr int n = rank2<A, B>::n > rank<C>::n ? rank2<A, B>::n : rank<C>::n;
};

// result containers by element kind and rank
template <int N> struct fres { using type = vf<N>; };
template <> struct fres<0> { using type = float; };
template <int N> struct ires { using type = vi<N>; };
template <> struct ires<0> { using type = long long; };
template <int N> struct bres { using type = vb<N>; };
template <> struct bres<0> { using type = bool; };

template <class T> struct is_intlike { static constexpr bool value = false; };
template <> struct is_intlike<int> { static constexpr bool value = true; };
template <> struct is_intlike<long> { static constexpr bool value = true; };
template <> struct is_intlike<long long> { static constexpr bool value = true; };
template <int N> struct is_intlike<vi<N>> { static constexpr bool value = true; };
template <class T> struct is_boollike { static constexpr bool value = false; };
template <> struct is_boollike<bool> { static constexpr bool value = true; };
template <int N> struct is_boollike<vb<N>> { static constexpr bool value = true; };

#define IXB_GEN_SET(res, i, val) \
  if constexpr (rank<decltype(res)>::n == 0) { res = (val); } else { res.v[i] = (val); }

// elementwise map helpers -------------------------------------------------------------
template <class R, class F, class A> __device__ __forceinline__ R map1(F f, const A& a) {
  constexpr int N = rank<R>::n;
  R r;
  if constexpr (N == 0) {
    r = f(at(a, 0));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = f(at(a, i));
  }
  return r;
}
template <class R, class F, class A, class B>
__device__ __forceinline__ R map2(F f, const A& a, const B& b) {
  constexpr int N = rank<R>::n;
  R r;
  if constexpr (N == 0) {
    r = f(at(a, 0), at(b, 0));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = f(at(a, i), at(b, i));
  }
  return r;
}
template <class R, class F, class A, class B, class C>
__device__ __forceinline__ R map3(F f, const A& a, const B& b, const C& c) {
  constexpr int N = rank<R>::n;
  R r;
  if constexpr (N == 0) {
    r = f(at(a, 0), at(b, 0), at(c, 0));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = f(at(a, i), at(b, i), at(c, i));
  }
  return r;
}

// arithmetic result kind: int op int -> int, anything with a float -> float
template <class A, class B> struct arith {
  static constexpr int n = rank2<A, B>::n;
  static constexpr bool ints = (is_intlike<A>::value || is_boollike<A>::value) &&
                               (is_intlike<B>::value || is_boollike<B>::value);
  using type = typename std::conditional<ints, typename ires<n>::type, typename fres<n>::type>::type;
  using elem = typename std::conditional<ints, long long, float>::type;
};

template <class T> struct is_vec { static constexpr bool value = rank<T>::n > 0; };
#define IXB_GEN_ANYVEC(A, B) typename std::enable_if<is_vec<A>::value || is_vec<B>::value, int>::type = 0

#define IXB_GEN_BINOP(OP)                                                                      \
  template <class A, class B, IXB_GEN_ANYVEC(A, B)>                                            \
  __device__ __forceinline__ typename arith<A, B>::type operator OP(const A& a, const B& b) {  \
    using E = typename arith<A, B>::elem;                                                      \
    return map2<typename arith<A, B>::type>([](E x, E y) { return x OP y; }, a, b);            \
  }
IXB_GEN_BINOP(+)
IXB_GEN_BINOP(-)
IXB_GEN_BINOP(*)
#undef IXB_GEN_BINOP

#define IXB_GEN_CMPOP(OP)                                                                       \
  template <class A, class B, IXB_GEN_ANYVEC(A, B)>                                             \
  __device__ __forceinline__ typename bres<rank2<A, B>::n>::type operator OP(const A& a,        \
                                                                              const B& b) {     \
    using E = typename arith<A, B>::elem;                                                       \
    return map2<typename bres<rank2<A, B>::n>::type>([](E x, E y) { return x OP y; }, a, b);    \
  }
IXB_GEN_CMPOP(<)
IXB_GEN_CMPOP(<=)
IXB_GEN_CMPOP(>)
IXB_GEN_CMPOP(>=)
IXB_GEN_CMPOP(==)
IXB_GEN_CMPOP(!=)
#undef IXB_GEN_CMPOP

template <class A, typename std::enable_if<is_vec<A>::value, int>::type = 0>
__device__ __forceinline__ A operator-(const A& a) {
  using E = typename std::conditional<is_intlike<A>::value, long long, float>::type;
  return map1<A>([](E x) { return -x; }, a);
}

}  // namespace gen
}  // namespace ixb
