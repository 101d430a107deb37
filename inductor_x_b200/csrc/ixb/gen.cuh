// Kernel templates instantiated by generated functor modules.  The code generator
// classifies a fused node group into one of these families and emits a `Body` struct
// whose single method is straight-line code over gen_vec / gen_ops types:
//
//   pointwise_gen_kernel<Body>   Body::tile(xbase, nvalid): kVec consecutive elements of
//                                the flattened iteration space per call (128-bit access
//                                where an operand is contiguous along it)
//   row_gen_kernel<Body,...>     Body::row(ctx, x): one reduced row held in the registers of
//                                a team (same work split as row.cuh)
//   outer_gen_kernel<Body,...>   Body::tile(ctx, xbase, nvalid): reductions whose reduced axis
//                                is not stride-1; threads map along the kept axis and the
//                                body loops over the reduced index
//
// They play the role of the decorators the reference attaches to every emitted kernel,
// pointwise_npu_index / persistent_reduction_npu_index / reduction_npu_index
// (inductor_x/npu_triton_heuristics.py:545-611).
#pragma once
#include "gen_ops.cuh"
#include "row.cuh"

namespace ixb {
namespace gen {

// ---- element access by storage type -------------------------------------------------
template <class T> struct Mem;
template <> struct Mem<float> {
  using val = float;
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
};
template <> struct Mem<f16> {
  using val = float;
  static __device__ __forceinline__ float ld(const f16* p) { return __half2float(*p); }
  static __device__ __forceinline__ void st(f16* p, float v) { *p = __float2half_rn(v); }
};
template <> struct Mem<bf16> {
  using val = float;
  static __device__ __forceinline__ float ld(const bf16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Mem<double> {
  using val = float;
  static __device__ __forceinline__ float ld(const double* p) { return (float)*p; }
  static __device__ __forceinline__ void st(double* p, float v) { *p = (double)v; }
};
template <> struct Mem<long long> {
  using val = long long;
  static __device__ __forceinline__ long long ld(const long long* p) { return *p; }
  static __device__ __forceinline__ void st(long long* p, long long v) { *p = v; }
};
template <> struct Mem<int> {
  using val = long long;
  static __device__ __forceinline__ long long ld(const int* p) { return *p; }
  static __device__ __forceinline__ void st(int* p, long long v) { *p = (int)v; }
};
template <> struct Mem<short> {
  using val = long long;
  static __device__ __forceinline__ long long ld(const short* p) { return *p; }
  static __device__ __forceinline__ void st(short* p, long long v) { *p = (short)v; }
};
template <> struct Mem<signed char> {
  using val = long long;
  static __device__ __forceinline__ long long ld(const signed char* p) { return *p; }
  static __device__ __forceinline__ void st(signed char* p, long long v) { *p = (signed char)v; }
};
template <> struct Mem<unsigned char> {
  using val = long long;
  static __device__ __forceinline__ long long ld(const unsigned char* p) { return *p; }
  static __device__ __forceinline__ void st(unsigned char* p, long long v) { *p = (unsigned char)v; }
};
template <> struct Mem<bool> {
  using val = bool;
  static __device__ __forceinline__ bool ld(const bool* p) { return *p; }
  static __device__ __forceinline__ void st(bool* p, bool v) { *p = v; }
};

template <class V, int N> struct vec_of;
template <int N> struct vec_of<float, N> { using type = typename fres<N>::type; };
template <int N> struct vec_of<long long, N> { using type = typename ires<N>::type; };
template <int N> struct vec_of<bool, N> { using type = typename bres<N>::type; };

// conversions the store side needs: any value kind -> the element kind of the buffer
template <class V> struct Cast;
template <> struct Cast<float> {
  static __device__ __forceinline__ float from(float v) { return v; }
  static __device__ __forceinline__ float from(double v) { return (float)v; }
  static __device__ __forceinline__ float from(long long v) { return (float)v; }
  static __device__ __forceinline__ float from(bool v) { return v ? 1.f : 0.f; }
};
template <> struct Cast<long long> {
  static __device__ __forceinline__ long long from(float v) { return (long long)v; }
  static __device__ __forceinline__ long long from(double v) { return (long long)v; }
  static __device__ __forceinline__ long long from(long long v) { return v; }
  static __device__ __forceinline__ long long from(bool v) { return v ? 1 : 0; }
};
template <> struct Cast<bool> {
  static __device__ __forceinline__ bool from(float v) { return v != 0.f; }
  static __device__ __forceinline__ bool from(double v) { return v != 0.0; }
  static __device__ __forceinline__ bool from(long long v) { return v != 0; }
  static __device__ __forceinline__ bool from(bool v) { return v; }
};

// iota: xbase, xbase+1, ...
template <int N> __device__ __forceinline__ vi<N> iota(long long base) {
  vi<N> r;
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = base + i;
  return r;
}
template <class A> __device__ __forceinline__ auto lane0(const A& a) { return at(a, 0); }

// gather: one scalar access per element, predicated by `mask` (false -> `other`)
template <class T, class I, class M>
__device__ __forceinline__ auto gather(const T* p, const I& idx, const M& mask,
                                       typename Mem<T>::val other) {
  using V = typename Mem<T>::val;
  constexpr int N = rank2<I, M>::n;
  typename vec_of<V, N>::type r;
  if constexpr (N == 0) {
    r = at(mask, 0) ? Mem<T>::ld(p + at(idx, 0)) : other;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = at(mask, i) ? Mem<T>::ld(p + at(idx, i)) : other;
  }
  return r;
}
template <class T, class I, class M, class A>
__device__ __forceinline__ void scatter(T* p, const I& idx, const M& mask, const A& val) {
  using V = typename Mem<T>::val;
  constexpr int N = rank3<I, M, A>::n;
  if constexpr (N == 0) {
    if (at(mask, 0)) Mem<T>::st(p + at(idx, 0), Cast<V>::from(at(val, 0)));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (at(mask, i)) Mem<T>::st(p + at(idx, i), Cast<V>::from(at(val, i)));
  }
}

// contiguous run of N elements starting at p: 128-bit accesses when the address allows
template <class T, int N>
__device__ __forceinline__ typename vec_of<typename Mem<T>::val, N>::type ldvec(const T* p, int nvalid) {
  using V = typename Mem<T>::val;
  typename vec_of<V, N>::type r;
  constexpr int kPer = 16 / sizeof(T);
  if constexpr ((N % kPer) == 0 && (sizeof(T) == 2 || sizeof(T) == 4) && std::is_same<V, float>::value) {
    if (nvalid >= N && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
#pragma unroll
      for (int c = 0; c < N / kPer; ++c) unpack<T>(ldg_keep(p + c * kPer), &r.v[c * kPer]);
      return r;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = i < nvalid ? Mem<T>::ld(p + i) : V();
  return r;
}
template <class T, int N, class A> __device__ __forceinline__ void stvec(T* p, int nvalid, const A& val) {
  using V = typename Mem<T>::val;
  constexpr int kPer = 16 / sizeof(T);
  if constexpr ((N % kPer) == 0 && (sizeof(T) == 2 || sizeof(T) == 4) && std::is_same<V, float>::value) {
    if (nvalid >= N && (reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
      float f[N];
#pragma unroll
      for (int i = 0; i < N; ++i) f[i] = Cast<float>::from(at(val, i));
#pragma unroll
      for (int c = 0; c < N / kPer; ++c) stg_stream(p + c * kPer, pack<T>(&f[c * kPer]));
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i)
    if (i < nvalid) Mem<T>::st(p + i, Cast<V>::from(at(val, i)));
}

// ---- pointwise family -------------------------------------------------------------------
template <class Body>
__global__ void __launch_bounds__(256) pointwise_gen_kernel(const Body body, const long long xnumel) {
  constexpr int V = Body::kVec;
  const long long ntiles = (xnumel + V - 1) / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ntiles; t += stride) {
    const long long xbase = t * V;
    const long long left = xnumel - xbase;
    body.tile(xbase, left >= V ? V : (int)left);
  }
}
template <class Body> int launch_pointwise(const Body& body, long long xnumel, void* stream) {
  if (xnumel <= 0) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long ntiles = (xnumel + Body::kVec - 1) / Body::kVec;
  long long grid = (ntiles + 255) / 256;
  const long long cap = (long long)sms * 16;  // persistent beyond 16 CTAs per SM
  if (grid > cap) grid = cap;
  pointwise_gen_kernel<Body><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(body, xnumel);
  return (int)cudaGetLastError();
}

// ---- persistent row family ---------------------------------------------------------------
// The generated body sees a context that maps vector element e = i * kVec + j of this
// thread to column vec_col(i) + j of the row, exactly as RowCtx does for the prebuilt bodies.
template <typename T, int TEAM, int TEAMS, int VPT> struct GenRowCtx : RowCtx<T, TEAM, TEAMS, VPT, false> {
  using Base = RowCtx<T, TEAM, TEAMS, VPT, false>;
  static constexpr int kE = VPT * Base::kVec;

  __device__ __forceinline__ vi<kE> rindex() const {
    vi<kE> r;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) r.v[i * Base::kVec + j] = this->vec_col(i) + j;
    return r;
  }
  __device__ __forceinline__ vb<kE> rmask() const {
    vb<kE> r;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) r.v[i * Base::kVec + j] = this->vec_col(i) + j < this->cols;
    return r;
  }
  // row-contiguous operand of storage type U starting at `rowp`
  template <class U> __device__ __forceinline__ auto load_row(const U* rowp) const {
    using V = typename Mem<U>::val;
    typename vec_of<V, kE>::type r;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c0 = this->vec_col(i);
      const int left = this->cols - c0;
      auto part = ldvec<U, Base::kVec>(rowp + c0, left > 0 ? left : 0);
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) r.v[i * Base::kVec + j] = part.v[j];
    }
    return r;
  }
  template <class U, class A> __device__ __forceinline__ void store_row(U* rowp, const A& val) const {
    using V = typename Mem<U>::val;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c0 = this->vec_col(i);
      const int left = this->cols - c0;
      typename vec_of<V, Base::kVec>::type part;
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) part.v[j] = Cast<V>::from(at(val, i * Base::kVec + j));
      stvec<U, Base::kVec>(rowp + c0, left > 0 ? left : 0, part);
    }
  }
  // reductions over the valid elements of the row
  template <class Op, class A> __device__ __forceinline__ float reduce(const A& val) {
    float acc = Op::identity();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (this->vec_col(i) + j < this->cols)
          acc = Op::combine(acc, Cast<float>::from(at(val, i * Base::kVec + j)));
    return Base::template reduce<Op>(acc);
  }
  template <bool IS_MAX, class A> __device__ __forceinline__ long long reduce_arg(const A& val) {
    ArgPair best = ArgOp<IS_MAX>::identity();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (this->vec_col(i) + j < this->cols)
          best = ArgOp<IS_MAX>::combine(
              best, ArgPair{Cast<float>::from(at(val, i * Base::kVec + j)), (long long)(this->vec_col(i) + j)});
    return Base::template reduce_arg<IS_MAX>(best).i;
  }
  template <class A> __device__ __forceinline__ bool reduce_any(const A& val) {
    return reduce<MaxOp>(op::where(val, 1.f, 0.f)) != 0.f;
  }
};

template <class Body, typename T, int TEAM, int TEAMS, int VPT>
__global__ void __launch_bounds__(TEAM* TEAMS)
    row_gen_kernel(const Body body, const long long rows, const int cols) {
  using Ctx = GenRowCtx<T, TEAM, TEAMS, VPT>;
  __shared__ __align__(16) float exchange[TEAMS * 2 * (TEAM / 32) * 4];
  Ctx c;
  c.lane = threadIdx.x % TEAM;
  c.team = threadIdx.x / TEAM;
  c.cols = cols;
  c.phase = 0;
  c.red = exchange + c.team * 2 * (TEAM / 32) * 4;
  const long long stride = (long long)gridDim.x * TEAMS;
  for (long long r = (long long)blockIdx.x * TEAMS + c.team; r < rows; r += stride) body.row(c, r);
}
template <class Body, typename T, int TEAM, int TEAMS, int VPT>
int launch_row_gen(const Body& body, long long rows, int cols, void* stream) {
  if (rows <= 0) return 0;
  auto kern = row_gen_kernel<Body, T, TEAM, TEAMS, VPT>;
  static int resident = 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (resident == 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, TEAM * TEAMS, 0) != cudaSuccess || n < 1) n = 1;
    resident = n;
  }
  const long long groups = (rows + TEAMS - 1) / TEAMS;
  long long grid = (long long)sms * resident;
  if (grid > groups) grid = groups;
  kern<<<(unsigned)grid, TEAM * TEAMS, 0, (cudaStream_t)stream>>>(body, rows, cols);
  return (int)cudaGetLastError();
}

// ---- outer reduction family -----------------------------------------------------------------
// The kept (x) axis is stride-1 in memory and the reduced axis is not: threads map along x
// (kVec consecutive elements each, a warp covers 32 * kVec of them) and the TY thread rows
// of a CTA split the reduced axis; their partial vectors are folded through shared memory.
// The generated body carries the loop over the reduced index itself:
//   Body::tile(ctx, xbase, nvalid)  - for (r = ctx.ty; r < rnumel; r += kTY) {...}, then
//                                     ctx.combine<Op>(acc), epilogue, stores by ty == 0.
template <int V, int TX, int TY> struct OuterCtx {
  static constexpr int kTY = TY;
  int tx, ty;
  float* part;  // [TY][TX * V]

  template <int N> static __device__ __forceinline__ vf<N> splat(float v) {
    vf<N> r;
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = v;
    return r;
  }
  // fold the TY partial vectors; every thread row receives the result
  template <class Op> __device__ __forceinline__ vf<V> combine(const vf<V>& acc) {
#pragma unroll
    for (int i = 0; i < V; ++i) part[(ty * TX + tx) * V + i] = acc.v[i];
    __syncthreads();
    vf<V> r;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float a = part[tx * V + i];
#pragma unroll
      for (int y = 1; y < TY; ++y) a = Op::combine(a, part[(y * TX + tx) * V + i]);
      r.v[i] = a;
    }
    __syncthreads();
    return r;
  }
};

template <class Body, int TX, int TY>
__global__ void __launch_bounds__(TX* TY) outer_gen_kernel(const Body body, const long long xnumel) {
  constexpr int V = Body::kVec;
  __shared__ float part[TY * TX * V];
  OuterCtx<V, TX, TY> c;
  c.tx = threadIdx.x % TX;
  c.ty = threadIdx.x / TX;
  c.part = part;
  const long long per_cta = (long long)TX * V;
  const long long ntiles = (xnumel + per_cta - 1) / per_cta;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long xbase = t * per_cta + (long long)c.tx * V;
    const long long left = xnumel - xbase;
    body.tile(c, xbase, left >= V ? V : (left > 0 ? (int)left : 0));
  }
}
template <class Body> int launch_outer_gen(const Body& body, long long xnumel, void* stream) {
  if (xnumel <= 0) return 0;
  constexpr int TX = 32, TY = 8;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long per_cta = (long long)TX * Body::kVec;
  long long grid = (xnumel + per_cta - 1) / per_cta;
  const long long cap = (long long)sms * 8;
  if (grid > cap) grid = cap;
  outer_gen_kernel<Body, TX, TY><<<(unsigned)grid, TX * TY, 0, (cudaStream_t)stream>>>(body, xnumel);
  return (int)cudaGetLastError();
}

}  // namespace gen
}  // namespace ixb
