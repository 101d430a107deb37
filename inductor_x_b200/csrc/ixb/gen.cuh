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

// contiguous run of N elements starting at p: 128-bit accesses when the address allows.
// FAST: the caller knows the run is complete and 16-byte aligned (full tile, aligned base
// pointer checked on the host, index proven a multiple of the vector), so the access is
// unconditional - no branch separates the loads of an unrolled loop and they overlap.
template <class T, int N, bool FAST = false>
__device__ __forceinline__ typename vec_of<typename Mem<T>::val, N>::type ldvec(const T* p, int nvalid) {
  using V = typename Mem<T>::val;
  typename vec_of<V, N>::type r;
  constexpr int kPer = 16 / sizeof(T);
  if constexpr ((N % kPer) == 0 && (sizeof(T) == 2 || sizeof(T) == 4) && std::is_same<V, float>::value) {
    if (FAST || (nvalid >= N && (reinterpret_cast<uintptr_t>(p) & 15u) == 0)) {
#pragma unroll
      for (int c = 0; c < N / kPer; ++c) unpack<T>(ldg_keep(p + c * kPer), &r.v[c * kPer]);
      return r;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = i < nvalid ? Mem<T>::ld(p + i) : V();
  return r;
}
template <class T, int N, bool FAST = false, class A>
__device__ __forceinline__ void stvec(T* p, int nvalid, const A& val) {
  using V = typename Mem<T>::val;
  constexpr int kPer = 16 / sizeof(T);
  if constexpr ((N % kPer) == 0 && (sizeof(T) == 2 || sizeof(T) == 4) && std::is_same<V, float>::value) {
    if (FAST || (nvalid >= N && (reinterpret_cast<uintptr_t>(p) & 15u) == 0)) {
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

// One element shared by all the elements a thread owns (an index or a per-row scale whose
// address does not change inside a vector): a single load, returned as a scalar, so that
// everything computed from it is scalar too.
template <class T>
__device__ __forceinline__ typename Mem<T>::val ld_uniform(const T* p, long long idx, bool valid,
                                                           typename Mem<T>::val other) {
  return valid ? Mem<T>::ld(p + idx) : other;
}
// Indirect access whose direct part is contiguous along the vector.  If every indirect
// operand turned out to be a scalar (it came from ld_uniform), the N elements are adjacent
// and move as one 128-bit access; otherwise one access per element.
template <class T, int N, bool FAST, class I, class M, class... U>
__device__ __forceinline__ auto igather(const T* p, const I& idx, const M& mask, typename Mem<T>::val other,
                                        int nvalid, const U&... indirect) {
  if constexpr (((rank<U>::n == 0) && ...) && rank<I>::n == N) {
    return ldvec<T, N, FAST>(p + at(idx, 0), nvalid);
  } else {
    return gather(p, idx, mask, other);
  }
}

// ---- pointwise family -------------------------------------------------------------------
// CTAs of `kern` that fit on the device at once.  Persistent kernels launch exactly this
// many (or fewer, if the work is smaller): a grid of a few waves would leave the last wave
// partly empty.
template <class K> inline long long resident_ctas(K kern, int threads) {
  int dev = 0, sms = 148, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, 0) != cudaSuccess || n < 1) n = 1;
  return (long long)sms * n;
}

// true when every pointer argument of a generated module is 16-byte aligned
inline bool pointers_aligned(void* const* ptrs, int n) {
  for (int i = 0; i < n; ++i)
    if (reinterpret_cast<uintptr_t>(ptrs[i]) & 15u) return false;
  return true;
}

template <class Body, bool ALIGNED>
__global__ void __launch_bounds__(256) pointwise_gen_kernel(const Body body, const long long xnumel) {
  constexpr int V = Body::kVec;
  const long long ntiles = (xnumel + V - 1) / V;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ntiles; t += stride) {
    const long long xbase = t * V;
    const long long left = xnumel - xbase;
    if (ALIGNED && left >= V) body.template tile<true>(xbase, V);
    else body.template tile<false>(xbase, left >= V ? V : (int)left);
  }
}
template <class Body> int launch_pointwise(const Body& body, long long xnumel, void* stream, bool aligned = false) {
  if (xnumel <= 0) return 0;
  static const long long cap_a = resident_ctas(pointwise_gen_kernel<Body, true>, 256);
  static const long long cap_u = resident_ctas(pointwise_gen_kernel<Body, false>, 256);
  const long long ntiles = (xnumel + Body::kVec - 1) / Body::kVec;
  long long grid = (ntiles + 255) / 256;
  const long long cap = aligned ? cap_a : cap_u;
  if (grid > cap) grid = cap;
  if (aligned) pointwise_gen_kernel<Body, true><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(body, xnumel);
  else pointwise_gen_kernel<Body, false><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(body, xnumel);
  return (int)cudaGetLastError();
}

// ---- persistent row family ---------------------------------------------------------------
// The generated body sees a context that maps vector element e = i * kVec + j of this
// thread to column vec_col(i) + j of the row, exactly as RowCtx does for the prebuilt bodies.
// FULL: the row fills every vector of the team exactly (length == TEAM * VPT * kVec), so no
// element needs a validity test.
template <typename T, int TEAM, int TEAMS, int VPT, bool FULL = false>
struct GenRowCtx : RowCtx<T, TEAM, TEAMS, VPT, false> {
  using Base = RowCtx<T, TEAM, TEAMS, VPT, false>;
  static constexpr int kE = VPT * Base::kVec;
  static constexpr int kGroup = TEAM < 32 ? TEAM : 32;  // lanes of one warp that share a row
  // Teams narrower than a warp share their warp's control flow: a team whose row index
  // ran past the end repeats the last row with `live` false, which masks its stores.
  bool live = true;

  __device__ __forceinline__ bool leader() const { return this->lane == 0 && live; }
  // element j of vector i lies inside the row
  __device__ __forceinline__ bool inside(int i, int j) const {
    return FULL ? true : (this->vec_col(i) + j < this->cols);
  }
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
      for (int j = 0; j < Base::kVec; ++j) r.v[i * Base::kVec + j] = live && inside(i, j);
    return r;
  }
  // row-contiguous operand of storage type U starting at `rowp`
  template <class U> __device__ __forceinline__ auto load_row(const U* rowp) const {
    using V = typename Mem<U>::val;
    typename vec_of<V, kE>::type r;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c0 = this->vec_col(i);
      const int left = FULL ? Base::kVec : this->cols - c0;
      auto part = ldvec<U, Base::kVec>(rowp + c0, left > 0 ? left : 0);
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) r.v[i * Base::kVec + j] = part.v[j];
    }
    return r;
  }
  // ask L2 for the lines of a row-contiguous operand this thread will load later: the
  // thread whose vector opens a 128-byte line (or the row itself) issues the prefetch
  template <class U> __device__ __forceinline__ void prefetch_row(const U* rowp) const {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c0 = this->vec_col(i);
      const U* p = rowp + c0;
      const bool opens = (reinterpret_cast<unsigned long long>(p) & 127ull) < Base::kVec * sizeof(U) || c0 == 0;
      if (c0 < this->cols && opens) asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
    }
  }
  template <class U, class A> __device__ __forceinline__ void store_row(U* rowp, const A& val) const {
    using V = typename Mem<U>::val;
    if (!live) return;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c0 = this->vec_col(i);
      const int left = FULL ? Base::kVec : this->cols - c0;
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
        if (inside(i, j))
          acc = Op::combine(acc, Cast<float>::from(at(val, i * Base::kVec + j)));
    if constexpr (TEAM < 32) return lane_group_reduce<Op, TEAM>(acc);
    else return Base::template reduce<Op>(acc);
  }
  template <bool IS_MAX, class A> __device__ __forceinline__ long long reduce_arg(const A& val) {
    ArgPair best = ArgOp<IS_MAX>::identity();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j))
          best = ArgOp<IS_MAX>::combine(
              best, ArgPair{Cast<float>::from(at(val, i * Base::kVec + j)), (long long)(this->vec_col(i) + j)});
    if constexpr (TEAM < 32) {
#pragma unroll
      for (int o = TEAM / 2; o > 0; o >>= 1) {
        ArgPair q;
        q.v = __shfl_xor_sync(kFull, best.v, o);
        q.i = __shfl_xor_sync(kFull, best.i, o);
        best = ArgOp<IS_MAX>::combine(best, q);
      }
      return best.i;
    } else {
      return Base::template reduce_arg<IS_MAX>(best).i;
    }
  }
  // (row maximum, sum of exp(value - maximum)) with a single exchange: every thread sums
  // relative to its own maximum and the partial sums are rescaled as they are folded
  struct MaxSum {
    float max, sum;
  };
  template <class A> __device__ __forceinline__ MaxSum online_softmax(const A& val) {
    constexpr float kLog2e = 1.4426950408889634f;
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j)) m = fmaxf(m, Cast<float>::from(at(val, i * Base::kVec + j)));
    if constexpr (TEAM < 32) m = lane_group_reduce<MaxOp, TEAM>(m);  // no exchange to save: plain two-step
    float s[1] = {0.f}, none[1] = {0.f};
    const float shift = (m == -INFINITY) ? 0.f : m;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j))
          s[0] += fast_exp2((Cast<float>::from(at(val, i * Base::kVec + j)) - shift) * kLog2e);
    if constexpr (TEAM < 32) s[0] = lane_group_reduce<SumOp, TEAM>(s[0]);
    else Base::template reduce_rescaled<1, 0>(m, s, none, kLog2e);
    return MaxSum{m, s[0]};
  }
  // (mean, sum of squared deviations, count) of the row with a single exchange: each
  // thread forms the statistics of its own elements and partial statistics are merged
  // pairwise (Chan et al.), which stays accurate when the mean is large against the spread
  struct Welford {
    float mean, m2, weight;
  };
  static __device__ __forceinline__ Welford merge(const Welford& a, const Welford& b) {
    const float n = a.weight + b.weight;
    const float w = n > 0.f ? __fdividef(b.weight, n) : 0.f;
    const float d = b.mean - a.mean;
    return Welford{fmaf(d, w, a.mean), a.m2 + b.m2 + d * d * a.weight * w, n};
  }
  template <class A> __device__ __forceinline__ Welford welford(const A& val) {
    float n = 0.f, sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j)) {
          n += 1.f;
          sum += Cast<float>::from(at(val, i * Base::kVec + j));
        }
    Welford w{n > 0.f ? sum / n : 0.f, 0.f, n};
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j)) {
          const float d = Cast<float>::from(at(val, i * Base::kVec + j)) - w.mean;
          w.m2 = fmaf(d, d, w.m2);
        }
#pragma unroll
    for (int off = kGroup / 2; off > 0; off >>= 1) {
      Welford o{__shfl_xor_sync(0xffffffffu, w.mean, off), __shfl_xor_sync(0xffffffffu, w.m2, off),
                __shfl_xor_sync(0xffffffffu, w.weight, off)};
      // both lanes of a pair must fold in the same order to agree bit for bit
      w = (this->lane & off) ? merge(o, w) : merge(w, o);
    }
    if constexpr (TEAM > 32) {
      float* slot = this->red + this->phase * Base::kWarpsPerTeam * 4;
      if ((this->lane & 31) == 0)
        *reinterpret_cast<float4*>(slot + (this->lane >> 5) * 4) = make_float4(w.mean, w.m2, w.weight, 0.f);
      team_barrier(this->team + 1, TEAM);
      const float4 first = *reinterpret_cast<const float4*>(slot);
      w = Welford{first.x, first.y, first.z};
#pragma unroll
      for (int k = 1; k < Base::kWarpsPerTeam; ++k) {
        const float4 part = *reinterpret_cast<const float4*>(slot + k * 4);
        w = merge(w, Welford{part.x, part.y, part.z});
      }
      this->phase ^= 1;
    }
    return w;
  }
  template <class A> __device__ __forceinline__ bool reduce_any(const A& val) {
    return reduce<MaxOp>(op::where(val, 1.f, 0.f)) != 0.f;
  }
};

template <class Body, typename T, int TEAM, int TEAMS, int VPT, int MIN_CTAS, int PF, bool FULL>
__global__ void __launch_bounds__(TEAM* TEAMS, MIN_CTAS)
    row_gen_kernel(const Body body, const long long rows, const int cols) {
  using Ctx = GenRowCtx<T, TEAM, TEAMS, VPT, FULL>;
  constexpr int kSlots = TEAM > 32 ? 2 * (TEAM / 32) * 4 : 1;  // exchange floats per team
  __shared__ __align__(16) float exchange[TEAMS * kSlots];
  Ctx c;
  c.lane = threadIdx.x % TEAM;
  c.team = threadIdx.x / TEAM;
  c.cols = cols;
  c.phase = 0;
  c.red = exchange + c.team * kSlots;
  const long long stride = (long long)gridDim.x * TEAMS;
  if constexpr (TEAM < 32) {
    // the teams of a warp run the same number of rows (full-mask shuffles inside)
    for (long long base = (long long)blockIdx.x * TEAMS; base < rows; base += stride) {
      const long long r = base + c.team;
      c.live = r < rows;
      body.row(c, c.live ? r : rows - 1);
    }
    return;
  }
  for (long long r = (long long)blockIdx.x * TEAMS + c.team; r < rows; r += stride) {
    // PF rows ahead of the one being worked on are on their way from DRAM to L2
    if constexpr (PF > 0) {
      const long long ahead = r + PF * stride;
      if (ahead < rows) body.prefetch(c, ahead);
    }
    body.row(c, r);
  }
}
template <class Body, typename T, int TEAM, int TEAMS, int VPT, int MIN_CTAS = 1, int PF = 0, bool FULL = false>
int launch_row_gen(const Body& body, long long rows, int cols, void* stream) {
  if (rows <= 0) return 0;
  if (FULL && cols != TEAM * VPT * Elem<T>::kVec) return (int)cudaErrorInvalidValue;
  auto kern = row_gen_kernel<Body, T, TEAM, TEAMS, VPT, MIN_CTAS, PF, FULL>;
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
// The kept (x) axis is stride-1 in memory and the reduced axis is not.  Threads form a
// TX x TY grid: TX threads cover the contiguous run of the kept axis (kVec elements each;
// TX is chosen by the generator so that TX * kVec elements are adjacent in memory) and the
// TY thread rows split the reduced axis.  With a short run a warp therefore reads 32 / TX
// consecutive reduced indices, which are adjacent spans when the reduced stride equals the
// run.  Partial vectors are folded by shuffles inside a warp and through shared memory
// across warps.  The generated body carries the loop over the reduced index itself:
//   Body::tile<FAST>(ctx, xbase, nvalid)  - for (r = ctx.ty; r < rnumel; r += kTY) {...},
//                                           then ctx.combine<Op>(acc), epilogue, stores by
//                                           the thread row ty == 0.
template <int V, int TX, int TY> struct OuterCtx {
  static constexpr int kTY = TY;
  static constexpr int kWarps = TX * TY / 32;
  static constexpr int kRowsPerWarp = 32 / TX;   // thread rows that share a warp
  static_assert(TX <= 32 && 32 % TX == 0 && (TX * TY) % 32 == 0, "thread grid must tile warps");
  int tx, ty;
  float* part;  // [kWarps][TX * V]

  template <int N> static __device__ __forceinline__ vf<N> splat(float v) {
    vf<N> r;
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = v;
    return r;
  }
  // fold the TY partial vectors; every thread row receives the result
  template <class Op> __device__ __forceinline__ vf<V> combine(const vf<V>& acc) {
    vf<V> r = acc;
#pragma unroll
    for (int off = TX; off < 32; off <<= 1)
#pragma unroll
      for (int i = 0; i < V; ++i) r.v[i] = Op::combine(r.v[i], __shfl_xor_sync(kFull, r.v[i], off));
    if constexpr (kWarps > 1) {
      const int warp = (ty * TX + tx) >> 5;
      if (ty % kRowsPerWarp == 0) {
#pragma unroll
        for (int i = 0; i < V; ++i) part[(warp * TX + tx) * V + i] = r.v[i];
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float a = part[tx * V + i];
#pragma unroll
        for (int w = 1; w < kWarps; ++w) a = Op::combine(a, part[(w * TX + tx) * V + i]);
        r.v[i] = a;
      }
      __syncthreads();
    }
    return r;
  }
};

template <class Body, int TX, int TY, bool ALIGNED>
__global__ void __launch_bounds__(TX* TY) outer_gen_kernel(const Body body, const long long xnumel) {
  constexpr int V = Body::kVec;
  __shared__ __align__(16) float part[(TX * TY / 32) * TX * V];
  OuterCtx<V, TX, TY> c;
  c.tx = threadIdx.x % TX;
  c.ty = threadIdx.x / TX;
  c.part = part;
  const long long per_cta = (long long)TX * V;
  const long long ntiles = (xnumel + per_cta - 1) / per_cta;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long xbase = t * per_cta + (long long)c.tx * V;
    const long long left = xnumel - xbase;
    // the choice is uniform per CTA (the fold synchronises the whole CTA)
    if (ALIGNED && xnumel - t * per_cta >= per_cta) body.template tile<true>(c, xbase, V);
    else body.template tile<false>(c, xbase, left >= V ? V : (left > 0 ? (int)left : 0));
  }
}
template <class Body, int TX = 32>
int launch_outer_gen(const Body& body, long long xnumel, void* stream, bool aligned = false) {
  if (xnumel <= 0) return 0;
  constexpr int TY = 256 / TX;
  static const long long cap_a = resident_ctas(outer_gen_kernel<Body, TX, TY, true>, TX * TY);
  static const long long cap_u = resident_ctas(outer_gen_kernel<Body, TX, TY, false>, TX * TY);
  const long long per_cta = (long long)TX * Body::kVec;
  long long grid = (xnumel + per_cta - 1) / per_cta;
  const long long cap = aligned ? cap_a : cap_u;
  if (grid > cap) grid = cap;
  if (aligned) outer_gen_kernel<Body, TX, TY, true><<<(unsigned)grid, TX * TY, 0, (cudaStream_t)stream>>>(body, xnumel);
  else outer_gen_kernel<Body, TX, TY, false><<<(unsigned)grid, TX * TY, 0, (cudaStream_t)stream>>>(body, xnumel);
  return (int)cudaGetLastError();
}

}  // namespace gen
}  // namespace ixb
