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
#include <atomic>

#include "gen_ops.cuh"
#include "row.cuh"
#include "tma.cuh"

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

// scatter with accumulation (store mode "atomic_add": index_put(accumulate=True), scatter_add
// and the outer split of the reference, inductor_x/codegen/triton.py:904-905): one atomic add
// per valid element, in the storage type of the destination
__device__ __forceinline__ void atomic_add(float* p, float v) { atomicAdd(p, v); }
__device__ __forceinline__ void atomic_add(f16* p, float v) { atomicAdd(p, __float2half_rn(v)); }
__device__ __forceinline__ void atomic_add(bf16* p, float v) { atomicAdd(p, __float2bfloat16_rn(v)); }
__device__ __forceinline__ void atomic_add(double* p, float v) { atomicAdd(p, (double)v); }
__device__ __forceinline__ void atomic_add(long long* p, long long v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
}
__device__ __forceinline__ void atomic_add(int* p, long long v) { atomicAdd(p, (int)v); }
template <class T, class I, class M, class A>
__device__ __forceinline__ void scatter_add(T* p, const I& idx, const M& mask, const A& val) {
  using V = typename Mem<T>::val;
  constexpr int N = rank3<I, M, A>::n;
  if constexpr (N == 0) {
    if (at(mask, 0)) atomic_add(p + at(idx, 0), Cast<V>::from(at(val, 0)));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i)
      if (at(mask, i)) atomic_add(p + at(idx, i), Cast<V>::from(at(val, i)));
  }
}

// contiguous run of N elements starting at p: 128-bit accesses when the address allows.
// FAST: the caller knows the run is complete and 16-byte aligned (full tile, aligned base
// pointer checked on the host, index proven a multiple of the vector), so the access is
// unconditional - no branch separates the loads of an unrolled loop and they overlap.
// STREAM: the run is read once and nothing near it is (a gathered table row): no L1 allocation.
template <class T, int N, bool FAST = false, bool STREAM = false>
__device__ __forceinline__ typename vec_of<typename Mem<T>::val, N>::type ldvec(const T* p, int nvalid) {
  using V = typename Mem<T>::val;
  typename vec_of<V, N>::type r;
  constexpr int kPer = 16 / sizeof(T);
  if constexpr ((N % kPer) == 0 && (sizeof(T) == 2 || sizeof(T) == 4) && std::is_same<V, float>::value) {
    if (FAST || (nvalid >= N && (reinterpret_cast<uintptr_t>(p) & 15u) == 0)) {
#pragma unroll
      for (int c = 0; c < N / kPer; ++c) {
        if constexpr (STREAM) unpack<T>(ldg_stream(p + c * kPer), &r.v[c * kPer]);
        else unpack<T>(ldg_keep(p + c * kPer), &r.v[c * kPer]);  // may be re-read: keep in L1
      }
      return r;
    }
  }
#pragma unroll
  for (int i = 0; i < N; ++i) r.v[i] = i < nvalid ? Mem<T>::ld(p + i) : V();
  return r;
}
// A run of N elements as the raw 128-bit words it was loaded as: what a thread holds while
// several independent loads are in flight, before any of them is widened.
template <class T, int N> struct RawVec {
  static constexpr int kWords = N * (int)sizeof(T) / 16;
  static_assert(kWords >= 1 && kWords * 16 == N * (int)sizeof(T), "whole 128-bit words");
  uint4 q[kWords];
};
// complete, 16-byte aligned run (the caller has established both), read once: no L1 allocation
template <class T, int N> __device__ __forceinline__ RawVec<T, N> ldraw(const T* p) {
  RawVec<T, N> r;
#pragma unroll
  for (int c = 0; c < RawVec<T, N>::kWords; ++c) r.q[c] = ldg_stream(p + c * (16 / (int)sizeof(T)));
  return r;
}
// Placed after a batch of ldraw calls: the words of `raw` cannot be consumed before this
// point, and (volatile statements keep their order) this point comes after every load of the
// batch - so all of them are issued before the first result is waited for.
template <class T, int N> __device__ __forceinline__ void pin(RawVec<T, N>& raw) {
#pragma unroll
  for (int c = 0; c < RawVec<T, N>::kWords; ++c)
    asm volatile("" : "+r"(raw.q[c].x), "+r"(raw.q[c].y), "+r"(raw.q[c].z), "+r"(raw.q[c].w));
}
template <class T, int N>
__device__ __forceinline__ typename vec_of<typename Mem<T>::val, N>::type widen_raw(const RawVec<T, N>& raw) {
  typename vec_of<typename Mem<T>::val, N>::type r;
  constexpr int kPer = 16 / (int)sizeof(T);
#pragma unroll
  for (int c = 0; c < RawVec<T, N>::kWords; ++c) unpack<T>(raw.q[c], &r.v[c * kPer]);
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
    return ldvec<T, N, FAST, true>(p + at(idx, 0), nvalid);
  } else {
    return gather(p, idx, mask, other);
  }
}

// ---- bounds check of indirect indices (debug builds) ---------------------------------------
// A module generated with IXB_DEBUG_BOUNDS checks every data-dependent index against the
// extent it addresses (the reference asserts them on the device,
// inductor_x/codegen/triton.py:1666-1710).  A violation is counted, one offending value is
// kept, and the index is replaced by 0 so that the access stays inside the buffer; the
// launcher reads the two words after the launch and raises on the host.  Nothing traps.
#ifdef IXB_DEBUG_BOUNDS
static __device__ unsigned long long g_bounds_status[2];  // [violations, one offending index]
__device__ __forceinline__ long long checked_one(long long x, long long size) {
  if (x < 0 || x >= size) {
    atomicAdd(&g_bounds_status[0], 1ull);
    atomicExch(&g_bounds_status[1], (unsigned long long)x);
    return 0;
  }
  return x;
}
template <class I> __device__ __forceinline__ auto checked_index(const I& idx, long long size) {
  return map1<typename ires<rank<I>::n>::type>([size](long long x) { return checked_one(x, size); }, idx);
}
// host: fetch and clear the status words of this module (synchronises the device)
inline int read_bounds_status(unsigned long long* out) {
  cudaError_t e = cudaMemcpyFromSymbol(out, g_bounds_status, 2 * sizeof(unsigned long long));
  if (e != cudaSuccess) return (int)e;
  const unsigned long long zero[2] = {0ull, 0ull};
  return (int)cudaMemcpyToSymbol(g_bounds_status, zero, sizeof(zero));
}
#endif

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
    // Body::first_of maps the thread's slot to the first element of its vector: t * V, or the
    // transposing order (consecutive lanes along the axis the loads are contiguous in)
    const long long xbase = body.first_of(t);
    const long long left = xnumel - xbase;
    if (ALIGNED && left >= V) body.template tile<true>(xbase, V);
    else body.template tile<false>(xbase, left >= V ? V : (int)left);
  }
}
// ---- transposes: a register tile per thread ---------------------------------------------------
// A pointwise group that stores along the flat index but reads an operand that is contiguous
// along another digit C of it (a transpose) gives every thread a V x kC micro-tile of that
// operand: V 128-bit loads, each kC consecutive elements along C (one for each of the V
// positions of the thread's vector along the flat index), then kC output vectors - element ci
// of every loaded row is the operand of output vector ci.  Both sides move 128 bits per access
// and the extraction costs what widening a half would cost anyway.  Lanes are arranged 4 along
// the flat index by 8 along C, so a warp reads four full 128-byte lines per load instruction
// and writes 64-byte runs.  This is what the reference's second set of index variables and
// `.permute(1, 0)` on the tile are for (inductor_x/codegen/triton.py:856-888, 1303-1332).
template <class U, int V> struct TileRaw {
  static constexpr int kC = 16 / (int)sizeof(U);
  uint4 q[V];
};
template <class U, int V, class I>
__device__ __forceinline__ void fetch_tile(TileRaw<U, V>& r, const U* p, const I& idx) {
#pragma unroll
  for (int j = 0; j < V; ++j) r.q[j] = ldg_stream(p + at(idx, j));
}
template <class U> __device__ __forceinline__ float tile_elem(const uint4& q, int ci);
template <> __device__ __forceinline__ float tile_elem<float>(const uint4& q, int ci) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  return __uint_as_float(w[ci]);
}
template <> __device__ __forceinline__ float tile_elem<bf16>(const uint4& q, int ci) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  return __uint_as_float((ci & 1) ? (w[ci >> 1] & 0xffff0000u) : (w[ci >> 1] << 16));
}
template <> __device__ __forceinline__ float tile_elem<f16>(const uint4& q, int ci) {
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
  const __half2 h = *reinterpret_cast<const __half2*>(&w[ci >> 1]);
  return (ci & 1) ? __high2float(h) : __low2float(h);
}
// element ci of every row of the tile, widened: the operand of output vector ci
template <class U, int V> __device__ __forceinline__ vf<V> take(const TileRaw<U, V>& t, int ci) {
  vf<V> r;
#pragma unroll
  for (int j = 0; j < V; ++j) r.v[j] = tile_elem<U>(t.q[j], ci);
  return r;
}

template <class Body>
__global__ void __launch_bounds__(256) pointwise_tile_gen_kernel(const Body body, const long long xnumel) {
  constexpr int V = Body::kVec;
  constexpr int C = Body::kTileC;
  const long long ntiles = xnumel / ((long long)V * C);     // exact by construction of the order
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < ntiles; t += stride) {
    const long long x0 = body.first_of_tile(t);
    typename Body::Tile raw;
    body.fetch_tile(x0, raw);
#pragma unroll
    for (int ci = 0; ci < C; ++ci) body.template tile<true, true>(x0 + ci * Body::kStepC, V, raw, ci);
  }
}
template <class Body> int launch_pointwise(const Body& body, long long xnumel, void* stream, bool aligned);
// tiles when every pointer is 16-byte aligned, the plain kernel (per-element gathers) otherwise
template <class Body> int launch_pointwise_tile(const Body& body, long long xnumel, void* stream, bool aligned) {
  if (xnumel <= 0) return 0;
  if (!aligned) return launch_pointwise(body, xnumel, stream, false);
  static const long long cap = resident_ctas(pointwise_tile_gen_kernel<Body>, 256);
  const long long ntiles = xnumel / ((long long)Body::kVec * Body::kTileC);
  long long grid = (ntiles + 255) / 256;
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  pointwise_tile_gen_kernel<Body><<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(body, xnumel);
  return (int)cudaGetLastError();
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
//
// A generated row body has four parts:
//   Consts / init(c, k)            operands that do not change from row to row (per-column
//                                  scales and shifts): loaded and widened once per thread
//   Raw / fetch(c, x, raw)         the 128-bit vectors of the operands streamed once per row,
//                                  requested one row ahead of the arithmetic
//   row<STAGED>(c, k, x, raw)      the math of row x; STAGED says whether `raw` was fetched
//                                  (aligned operands) or the body loads for itself
//   prefetch(c, x)                 L2 prefetch of the streamed operands of a later row

// raw 128-bit vectors of one row-shaped operand of storage type U, as one thread holds them
template <class U, int VPT, int KVEC> struct RawRow {
  static constexpr int kChunks = KVEC * (int)sizeof(U) / 16;  // 128-bit words per vector
  static_assert(kChunks >= 1, "staged operands are at least as wide as the row's vector type");
  uint4 q[VPT][kChunks];
};

// exact 64-bit integer reduction operators
struct ISum {
  static __device__ __forceinline__ long long id() { return 0; }
  static __device__ __forceinline__ long long f(long long a, long long b) { return a + b; }
};
struct IProd {
  static __device__ __forceinline__ long long id() { return 1; }
  static __device__ __forceinline__ long long f(long long a, long long b) { return a * b; }
};
struct IMax {
  static __device__ __forceinline__ long long id() { return (long long)0x8000000000000000ull; }
  static __device__ __forceinline__ long long f(long long a, long long b) { return a > b ? a : b; }
};
struct IMin {
  static __device__ __forceinline__ long long id() { return 0x7fffffffffffffffLL; }
  static __device__ __forceinline__ long long f(long long a, long long b) { return a < b ? a : b; }
};

// references to up to two float vectors (operands of the online-softmax riders)
template <int E, int K> struct VecRefs {
  const vf<E>* p[K > 0 ? K : 1];
};
template <int E> __device__ __forceinline__ VecRefs<E, 0> refs() { return VecRefs<E, 0>{{nullptr}}; }
template <int E> __device__ __forceinline__ VecRefs<E, 1> refs(const vf<E>& a) { return VecRefs<E, 1>{{&a}}; }
template <int E> __device__ __forceinline__ VecRefs<E, 2> refs(const vf<E>& a, const vf<E>& b) {
  return VecRefs<E, 2>{{&a, &b}};
}

// one warp-level sum of K values: every lane receives every total
template <int K> __device__ __forceinline__ void warp_sum(float (&v)[K]) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
#pragma unroll
    for (int k = 0; k < K; ++k) v[k] += __shfl_xor_sync(kFull, v[k], o);
}
// NaN-propagating maximum / minimum of a warp in one instruction
__device__ __forceinline__ float warp_max_nan(float v) {
  float r;
  asm volatile("redux.sync.max.NaN.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float warp_min_nan(float v) {
  float r;
  asm volatile("redux.sync.min.NaN.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
template <class Op> __device__ __forceinline__ float warp_all(float v) {
  if constexpr (std::is_same<Op, MaxOp>::value) return warp_max_nan(v);
  else if constexpr (std::is_same<Op, MinOp>::value) return warp_min_nan(v);
  else return warp_reduce<Op>(v);
}

template <typename T, int TEAM, int TEAMS, int VPT, bool FULL = false>
struct GenRowCtx : RowCtx<T, TEAM, TEAMS, VPT, false> {
  using Base = RowCtx<T, TEAM, TEAMS, VPT, false>;
  static constexpr int kE = VPT * Base::kVec;
  static constexpr int kGroup = TEAM < 32 ? TEAM : 32;  // lanes of one warp that share a row
  static constexpr int kW = Base::kWarpsPerTeam;        // warps per team (0 for sub-warp teams)
  static constexpr int kChains = (kE / 2) >= 4 ? 4 : ((kE / 2) >= 2 ? 2 : 1);  // accumulator chains
  // Teams narrower than a warp share their warp's control flow: a team whose row index
  // ran past the end repeats the last row with `live` false, which masks its stores.
  bool live = true;
  // Rows longer than the team holds are walked in chunks of kCap columns (looped reduction):
  // chunk0 is the first column of the current chunk.  vec_col shadows the base-class version,
  // so every access below is relative to the chunk.
  int chunk0 = 0;
  static constexpr int kCap = TEAM * VPT * Base::kVec;
  __device__ __forceinline__ int vec_col(int i) const { return chunk0 + (this->lane + i * TEAM) * Base::kVec; }
  __device__ __forceinline__ int nchunks() const { return (this->cols + kCap - 1) / kCap; }
  __device__ __forceinline__ void set_chunk(int chunk) { chunk0 = chunk * kCap; }
  // Per-column operands that are not kept in registers live in a CTA-wide shared-memory
  // table, widened to fp32 once at start-up.  Slot s is laid out [quad][vector] (a quad = four
  // floats) so that consecutive lanes read consecutive 16-byte words: no bank conflicts.
  const float4* ktab = nullptr;
  static constexpr int kQuads = Base::kVec / 4 > 0 ? Base::kVec / 4 : 1;
  static constexpr int kTabVecs = TEAM * VPT;   // vectors of one row at full capacity

  template <int SLOT, class U> __device__ __forceinline__ void fill_sconst(const U* rowp) const {
    static_assert(Base::kVec % 4 == 0, "shared-memory operands need whole quads per vector");
    float4* tab = const_cast<float4*>(ktab) + SLOT * kQuads * kTabVecs;
    for (int v = threadIdx.x; v < kTabVecs; v += blockDim.x) {
      const int c0 = v * Base::kVec;
      const int left = this->cols - c0;
      const auto part = ldvec<U, Base::kVec>(rowp + (left > 0 ? c0 : 0), left > 0 ? left : 0);
#pragma unroll
      for (int q = 0; q < kQuads; ++q)
        tab[q * kTabVecs + v] = make_float4(part.v[4 * q], part.v[4 * q + 1], part.v[4 * q + 2], part.v[4 * q + 3]);
    }
  }
  template <int SLOT> __device__ __forceinline__ vf<kE> sconst() const {
    const float4* tab = ktab + SLOT * kQuads * kTabVecs;
    vf<kE> r;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = this->lane + i * TEAM;
#pragma unroll
      for (int q = 0; q < kQuads; ++q) {
        const float4 f = tab[q * kTabVecs + v];
        r.v[i * Base::kVec + 4 * q] = f.x;
        r.v[i * Base::kVec + 4 * q + 1] = f.y;
        r.v[i * Base::kVec + 4 * q + 2] = f.z;
        r.v[i * Base::kVec + 4 * q + 3] = f.w;
      }
    }
    return r;
  }

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
  // the same operand as raw 128-bit vectors (aligned rows only; vectors past the end of a
  // ragged row read as zero): requested a row ahead, widened when the row is worked on
  template <class U> __device__ __forceinline__ void fetch_row(const U* rowp, RawRow<U, VPT, Base::kVec>& raw) const {
    constexpr int kC = RawRow<U, VPT, Base::kVec>::kChunks;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c0 = this->vec_col(i);
#pragma unroll
      for (int k = 0; k < kC; ++k)
        raw.q[i][k] = (FULL || c0 < this->cols) ? ldg_stream(reinterpret_cast<const uint4*>(rowp + c0) + k)
                                               : make_uint4(0, 0, 0, 0);
    }
  }
  template <class U> __device__ __forceinline__ vf<kE> widen(const RawRow<U, VPT, Base::kVec>& raw) const {
    constexpr int kC = RawRow<U, VPT, Base::kVec>::kChunks;
    constexpr int kPer = 16 / (int)sizeof(U);
    vf<kE> r;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int k = 0; k < kC; ++k) unpack<U>(raw.q[i][k], &r.v[i * Base::kVec + k * kPer]);
    return r;
  }
  // a streamed operand inside row(): from the fetched vectors, or loaded on the spot
  template <bool STAGED, class U>
  __device__ __forceinline__ vf<kE> operand(const RawRow<U, VPT, Base::kVec>& raw, const U* rowp) const {
    if constexpr (STAGED) return widen<U>(raw);
    else return load_row(rowp);
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
  // aligned rows: one 128-bit streaming store per vector, no address test
  template <bool STAGED, class U, class A> __device__ __forceinline__ void put_row(U* rowp, const A& val) const {
    if constexpr (STAGED && std::is_same<typename Mem<U>::val, float>::value && (sizeof(U) == 2 || sizeof(U) == 4) &&
                  std::is_same<A, vf<kE>>::value) {
      if (!live) return;
      constexpr int kPer = 16 / (int)sizeof(U);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c0 = this->vec_col(i);
        if (FULL || c0 < this->cols) {
#pragma unroll
          for (int k = 0; k < Base::kVec / kPer; ++k)
            stg_stream(rowp + c0 + k * kPer, pack<U>(&val.v[i * Base::kVec + k * kPer]));
        }
      }
    } else {
      store_row(rowp, val);
    }
  }

  // ---- team exchange --------------------------------------------------------------------
  // Partial results cross warps through one 16-byte slot per warp; after the team barrier
  // lane l of every warp reads the slot of warp l mod kW and a shuffle tree over kW lanes
  // folds them, so the cost per thread does not grow with the number of warps in the team.
  __device__ __forceinline__ float* slot_base() { return this->red + this->phase * kW * 4; }
  template <class Op> __device__ __forceinline__ float xreduce(float v) {
    if constexpr (TEAM < 32) {
      return lane_group_reduce<Op, TEAM>(v);
    } else {
      v = warp_all<Op>(v);
      if constexpr (kW > 1) {
        float* slot = slot_base();
        if ((this->lane & 31) == 0) slot[(this->lane >> 5) * 4] = v;
        team_barrier(this->team + 1, TEAM);
        v = slot[(this->lane & (kW - 1)) * 4];
        v = lane_group_reduce<Op, kW>(v);
        this->phase ^= 1;
      }
      return v;
    }
  }
  // K sums with one barrier (K <= 4)
  template <int K> __device__ __forceinline__ void xsum(float (&v)[K]) {
    static_assert(K <= 4, "a slot holds four floats");
    if constexpr (TEAM < 32) {
#pragma unroll
      for (int k = 0; k < K; ++k) v[k] = lane_group_reduce<SumOp, TEAM>(v[k]);
    } else {
      warp_sum<K>(v);
      if constexpr (kW > 1) {
        float* slot = slot_base();
        if ((this->lane & 31) == 0) {
#pragma unroll
          for (int k = 0; k < K; ++k) slot[(this->lane >> 5) * 4 + k] = v[k];
        }
        team_barrier(this->team + 1, TEAM);
        const float* mine = slot + (this->lane & (kW - 1)) * 4;
#pragma unroll
        for (int k = 0; k < K; ++k) v[k] = lane_group_reduce<SumOp, kW>(mine[k]);
        this->phase ^= 1;
      }
    }
  }

  // ---- inclusive prefix scan along the row (cumsum / cumprod over the stride-1 axis) -----------
  // Row order: vector i of thread t is vector i * TEAM + t of the row.  Per round i every
  // thread scans its own vector, the vector totals are scanned over the team in thread order
  // (shuffles inside a warp, one slot per warp across warps), and the total of the rounds
  // before is carried along.  Op is SumOp or ProdOp; fp32 accumulation, as the reference's sums.
  template <class Op, class A> __device__ __forceinline__ vf<kE> scan(const A& val) {
    vf<kE> out;
    float carry = Op::identity();
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      float run = Op::identity();
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) {
        run = Op::combine(run, inside(i, j) ? Cast<float>::from(at(val, i * Base::kVec + j)) : Op::identity());
        out.v[i * Base::kVec + j] = run;
      }
      // inclusive scan of `run` over the lanes of this thread's warp (or lane group), and the
      // exclusive one beside it (the operator need not have an inverse)
      float incl = run, before = Op::identity();
      const int wl = this->lane & (kGroup - 1);
#pragma unroll
      for (int off = 1; off < kGroup; off <<= 1) {
        const float up_i = __shfl_up_sync(kFull, incl, off, kGroup);
        if (wl >= off) incl = Op::combine(up_i, incl);
      }
      if constexpr (std::is_same<Op, SumOp>::value) {
        before = incl - run;              // sums have an inverse: no second shuffle
      } else {
        const float up = __shfl_up_sync(kFull, incl, 1, kGroup);
        if (wl >= 1) before = up;
      }
      float total = __shfl_sync(kFull, incl, kGroup - 1, kGroup);  // the warp's (group's) total
      if constexpr (TEAM > 32) {
        float* slot = slot_base();
        const int w = this->lane >> 5;
        if ((this->lane & 31) == 31) slot[w * 4] = incl;
        team_barrier(this->team + 1, TEAM);
        float ahead = Op::identity(), all = Op::identity();
#pragma unroll
        for (int k = 0; k < kW; ++k) {
          const float tk = slot[k * 4];
          if (k < w) ahead = Op::combine(ahead, tk);
          all = Op::combine(all, tk);
        }
        before = Op::combine(ahead, before);
        total = all;
        this->phase ^= 1;
      }
      const float base = Op::combine(carry, before);
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) out.v[i * Base::kVec + j] = Op::combine(base, out.v[i * Base::kVec + j]);
      carry = Op::combine(carry, total);
    }
    return out;
  }
  // the same scan with exact 64-bit integers (cumsum / cumprod of integer, index or boolean rows)
  template <class IOp, class A> __device__ __forceinline__ vi<kE> scan_int(const A& val) {
    vi<kE> out;
    long long carry = IOp::id();
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      long long run = IOp::id();
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) {
        run = IOp::f(run, inside(i, j) ? Cast<long long>::from(at(val, i * Base::kVec + j)) : IOp::id());
        out.v[i * Base::kVec + j] = run;
      }
      long long incl = run, before = IOp::id();
      const int wl = this->lane & (kGroup - 1);
#pragma unroll
      for (int off = 1; off < kGroup; off <<= 1) {
        const long long up_i = __shfl_up_sync(kFull, incl, off, kGroup);
        if (wl >= off) incl = IOp::f(up_i, incl);
      }
      if constexpr (std::is_same<IOp, ISum>::value) {
        before = incl - run;
      } else {
        const long long up = __shfl_up_sync(kFull, incl, 1, kGroup);
        if (wl >= 1) before = up;
      }
      long long total = __shfl_sync(kFull, incl, kGroup - 1, kGroup);
      if constexpr (TEAM > 32) {
        long long* slot = reinterpret_cast<long long*>(slot_base());
        const int w = this->lane >> 5;
        if ((this->lane & 31) == 31) slot[w * 2] = incl;
        team_barrier(this->team + 1, TEAM);
        long long ahead = IOp::id(), all = IOp::id();
#pragma unroll
        for (int k = 0; k < kW; ++k) {
          const long long tk = slot[k * 2];
          if (k < w) ahead = IOp::f(ahead, tk);
          all = IOp::f(all, tk);
        }
        before = IOp::f(ahead, before);
        total = all;
        this->phase ^= 1;
      }
      const long long base = IOp::f(carry, before);
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j) out.v[i * Base::kVec + j] = IOp::f(base, out.v[i * Base::kVec + j]);
      carry = IOp::f(carry, total);
    }
    return out;
  }

  // ---- thread-local folds -------------------------------------------------------------------
  template <class A> __device__ __forceinline__ float local_sum(const A& val) const {
    if constexpr (FULL && op::is_fvec<A>::value) {
      // kChains independent chains of packed adds: a single chain would serialise on the
      // add latency with only a few warps resident
      float2 acc[kChains];
#pragma unroll
      for (int c = 0; c < kChains; ++c) acc[c] = op::pr(val, c);
#pragma unroll
      for (int p = kChains; p < kE / 2; ++p) acc[p % kChains] = add2(acc[p % kChains], op::pr(val, p));
#pragma unroll
      for (int c = 1; c < kChains; ++c) acc[0] = add2(acc[0], acc[c]);
      return acc[0].x + acc[0].y;
    } else {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < Base::kVec; ++j)
          if (inside(i, j)) acc += Cast<float>::from(at(val, i * Base::kVec + j));
      return acc;
    }
  }
  // sum of a[e] * b[e]
  template <class A, class B> __device__ __forceinline__ float local_dot(const A& a, const B& b) const {
    if constexpr (FULL && op::packable2<A, B>::value) {
      float2 acc[kChains];
#pragma unroll
      for (int c = 0; c < kChains; ++c) acc[c] = mul2(op::pr(a, c), op::pr(b, c));
#pragma unroll
      for (int p = kChains; p < kE / 2; ++p) acc[p % kChains] = fma2(op::pr(a, p), op::pr(b, p), acc[p % kChains]);
#pragma unroll
      for (int c = 1; c < kChains; ++c) acc[0] = add2(acc[0], acc[c]);
      return acc[0].x + acc[0].y;
    } else {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < Base::kVec; ++j)
          if (inside(i, j))
            acc = fmaf(Cast<float>::from(at(a, i * Base::kVec + j)), Cast<float>::from(at(b, i * Base::kVec + j)), acc);
      return acc;
    }
  }
  template <class Op, class A> __device__ __forceinline__ float local_fold(const A& val) const {
    if constexpr (std::is_same<Op, SumOp>::value) {
      return local_sum(val);
    } else {
      float acc = Op::identity();
#pragma unroll
      for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int j = 0; j < Base::kVec; ++j)
          if (inside(i, j)) acc = Op::combine(acc, Cast<float>::from(at(val, i * Base::kVec + j)));
      return acc;
    }
  }

  // reductions over the valid elements of the row
  template <class Op, class A> __device__ __forceinline__ float reduce(const A& val) {
    return xreduce<Op>(local_fold<Op>(val));
  }
  // sum of an element-wise product (the multiply rides in the accumulating fma)
  template <class A, class B> __device__ __forceinline__ float reduce_dot(const A& a, const B& b) {
    return xreduce<SumOp>(local_dot(a, b));
  }
  // Exact integer reductions: 64-bit accumulators, shuffled as two halves, exchanged
  // through the same slots (a slot holds two 64-bit values).
  using ISum = ::ixb::gen::ISum;
  using IProd = ::ixb::gen::IProd;
  using IMax = ::ixb::gen::IMax;
  using IMin = ::ixb::gen::IMin;
  template <class IOp, class A> __device__ __forceinline__ long long local_fold_int(const A& val) const {
    long long acc = IOp::id();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j)) acc = IOp::f(acc, Cast<long long>::from(at(val, i * Base::kVec + j)));
    return acc;
  }
  template <class IOp> __device__ __forceinline__ long long xreduce_int(long long acc) {
#pragma unroll
    for (int o = kGroup / 2; o > 0; o >>= 1) acc = IOp::f(acc, __shfl_xor_sync(kFull, acc, o));
    if constexpr (kW > 1) {
      long long* slot = reinterpret_cast<long long*>(slot_base());
      if ((this->lane & 31) == 0) slot[(this->lane >> 5) * 2] = acc;
      team_barrier(this->team + 1, TEAM);
      acc = slot[(this->lane & (kW - 1)) * 2];
#pragma unroll
      for (int o = kW / 2; o > 0; o >>= 1) acc = IOp::f(acc, __shfl_xor_sync(kFull, acc, o));
      this->phase ^= 1;
    }
    return acc;
  }
  template <class IOp, class A> __device__ __forceinline__ long long reduce_int(const A& val) {
    return xreduce_int<IOp>(local_fold_int<IOp>(val));
  }
  template <bool IS_MAX, class A> __device__ __forceinline__ ArgPair local_arg(const A& val) const {
    ArgPair best = ArgOp<IS_MAX>::identity();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j))
          best = ArgOp<IS_MAX>::combine(
              best, ArgPair{Cast<float>::from(at(val, i * Base::kVec + j)), (long long)(vec_col(i) + j)});
    return best;
  }
  template <bool IS_MAX> __device__ __forceinline__ long long xreduce_arg(ArgPair best) {
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
  template <bool IS_MAX, class A> __device__ __forceinline__ long long reduce_arg(const A& val) {
    return xreduce_arg<IS_MAX>(local_arg<IS_MAX>(val));
  }

  // arg-reductions of 32- and 64-bit integers: compared as integers (as floats, neighbours
  // beyond 2^24 would tie and the smaller index would win); same tie rule, no NaN to consider
  struct ArgPairI {
    long long v, i;
  };
  template <bool IS_MAX> static __device__ __forceinline__ ArgPairI arg_identity_int() {
    return ArgPairI{IS_MAX ? (-0x7fffffffffffffffLL - 1) : 0x7fffffffffffffffLL, 0x7fffffffffffffffLL};
  }
  template <bool IS_MAX> static __device__ __forceinline__ ArgPairI arg_better(ArgPairI a, ArgPairI b) {
    const bool take_b = (a.v == b.v) ? (b.i < a.i) : (IS_MAX ? (b.v > a.v) : (b.v < a.v));
    return take_b ? b : a;
  }
  template <bool IS_MAX, class A> __device__ __forceinline__ ArgPairI local_arg_int(const A& val) const {
    ArgPairI best = arg_identity_int<IS_MAX>();
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j))
          best = arg_better<IS_MAX>(
              best, ArgPairI{Cast<long long>::from(at(val, i * Base::kVec + j)), (long long)(vec_col(i) + j)});
    return best;
  }
  template <bool IS_MAX> __device__ __forceinline__ long long xreduce_arg_int(ArgPairI best) {
#pragma unroll
    for (int o = kGroup / 2; o > 0; o >>= 1) {
      ArgPairI q;
      q.v = __shfl_xor_sync(kFull, best.v, o);
      q.i = __shfl_xor_sync(kFull, best.i, o);
      best = arg_better<IS_MAX>(best, q);
    }
    if constexpr (kW > 1) {
      long long* slot = reinterpret_cast<long long*>(slot_base());   // a slot holds the pair
      if ((this->lane & 31) == 0) {
        slot[(this->lane >> 5) * 2] = best.v;
        slot[(this->lane >> 5) * 2 + 1] = best.i;
      }
      team_barrier(this->team + 1, TEAM);
      best.v = slot[(this->lane & (kW - 1)) * 2];
      best.i = slot[(this->lane & (kW - 1)) * 2 + 1];
#pragma unroll
      for (int o = kW / 2; o > 0; o >>= 1) {
        ArgPairI q;
        q.v = __shfl_xor_sync(kFull, best.v, o);
        q.i = __shfl_xor_sync(kFull, best.i, o);
        best = arg_better<IS_MAX>(best, q);
      }
      this->phase ^= 1;
    }
    return best.i;
  }
  template <bool IS_MAX, class A> __device__ __forceinline__ long long reduce_arg_int(const A& val) {
    return xreduce_arg_int<IS_MAX>(local_arg_int<IS_MAX>(val));
  }

  // ---- online softmax ------------------------------------------------------------------------
  // One exchange yields the row maximum, the sum of exp(value - maximum) and up to three
  // further row sums ("riders") that the emitter found it could form before the maximum is
  // known: NS of them are sums of exp(value - maximum) * w for a vector w (they are
  // accumulated relative to each thread's own maximum and rescaled as partial results are
  // folded, like the sum itself), NP are ordinary sums.  The thread keeps its exponentials
  // relative to its own maximum in `e` and the factor `r` that brings them to the row
  // maximum, so that exp(value - maximum) costs one multiply afterwards instead of a second
  // pass over the exponential unit.
  template <int NS, int NP> struct Online {
    float max, sum, r;
    vf<kE> e;
    float scaled[NS > 0 ? NS : 1], plain[NP > 0 ? NP : 1];
  };
  template <int NS, int NP, class A>
  __device__ __forceinline__ Online<NS, NP> online_softmax(const A& val, const VecRefs<kE, NS>& w,
                                                            const VecRefs<kE, NP>& pl) {
    static_assert(NS + NP <= 2, "a slot holds the maximum, the sum and two riders");
    Online<NS, NP> o;
    float mc[kChains];
#pragma unroll
    for (int c = 0; c < kChains; ++c) mc[c] = -INFINITY;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; j += 2) {
        const int e0 = i * Base::kVec + j;
        const float a = inside(i, j) ? Cast<float>::from(at(val, e0)) : -INFINITY;
        const float b = inside(i, j + 1) ? Cast<float>::from(at(val, e0 + 1)) : -INFINITY;
        mc[(e0 / 2) % kChains] = max3(mc[(e0 / 2) % kChains], a, b);
      }
    float m = mc[0];
#pragma unroll
    for (int c = 1; c < kChains; ++c) m = fmaxf(m, mc[c]);
    // v[0] = sum of exponentials, v[1..NS] scaled riders, then the plain riders
    float v[1 + NS + NP];
#pragma unroll
    for (int k = 0; k < 1 + NS + NP; ++k) v[k] = 0.f;
    const float shift = (m == -INFINITY) ? 0.f : -m * kLog2e;
    float2 acc[1 + NS][kChains];
#pragma unroll
    for (int k = 0; k < 1 + NS; ++k)
#pragma unroll
      for (int c = 0; c < kChains; ++c) acc[k][c] = make_float2(0.f, 0.f);
#pragma unroll
    for (int p = 0; p < kE / 2; ++p) {
      const float2 x = make_float2(Cast<float>::from(at(val, 2 * p)), Cast<float>::from(at(val, 2 * p + 1)));
      const float2 t = fma2(x, make_float2(kLog2e, kLog2e), make_float2(shift, shift));
      float2 ex = make_float2(fast_exp2(t.x), fast_exp2(t.y));
      if constexpr (!FULL) {
        if (!inside((2 * p) / Base::kVec, (2 * p) % Base::kVec)) ex.x = 0.f;
        if (!inside((2 * p + 1) / Base::kVec, (2 * p + 1) % Base::kVec)) ex.y = 0.f;
      }
      o.e.v[2 * p] = ex.x;
      o.e.v[2 * p + 1] = ex.y;
      acc[0][p % kChains] = add2(acc[0][p % kChains], ex);
#pragma unroll
      for (int k = 0; k < NS; ++k) acc[1 + k][p % kChains] = fma2(ex, op::pr(*w.p[k], p), acc[1 + k][p % kChains]);
    }
#pragma unroll
    for (int k = 0; k < 1 + NS; ++k) {
#pragma unroll
      for (int c = 1; c < kChains; ++c) acc[k][0] = add2(acc[k][0], acc[k][c]);
      v[k] = acc[k][0].x + acc[k][0].y;
    }
#pragma unroll
    for (int k = 0; k < NP; ++k) v[1 + NS + k] = local_sum(*pl.p[k]);

    // warp stage: agree on the warp's maximum, rescale, sum
    float r;
    if constexpr (TEAM < 32) {
      const float mw = lane_group_reduce<FastMaxOp, TEAM>(m);
      r = (m == -INFINITY) ? 0.f : fast_exp2((m - mw) * kLog2e);
#pragma unroll
      for (int k = 0; k < 1 + NS; ++k) v[k] *= r;
#pragma unroll
      for (int k = 0; k < 1 + NS + NP; ++k) v[k] = lane_group_reduce<SumOp, TEAM>(v[k]);
      m = mw;
    } else {
      const float mw = warp_max_fast(m);
      r = (m == -INFINITY) ? 0.f : fast_exp2((m - mw) * kLog2e);
#pragma unroll
      for (int k = 0; k < 1 + NS; ++k) v[k] *= r;
      warp_sum<1 + NS + NP>(v);
      m = mw;
      if constexpr (kW > 1) {
        float* slot = slot_base();
        if ((this->lane & 31) == 0) {
          float4 s4 = make_float4(mw, v[0], 0.f, 0.f);
          if constexpr (1 + NS + NP > 1) s4.z = v[1];
          if constexpr (1 + NS + NP > 2) s4.w = v[2];
          *reinterpret_cast<float4*>(slot + (this->lane >> 5) * 4) = s4;
        }
        team_barrier(this->team + 1, TEAM);
        const float4 part = *reinterpret_cast<const float4*>(slot + (this->lane & (kW - 1)) * 4);
        const float mm = lane_group_reduce<FastMaxOp, kW>(part.x);
        const float f = (part.x == -INFINITY) ? 0.f : fast_exp2((part.x - mm) * kLog2e);
        const float pv[3] = {part.y, part.z, part.w};
#pragma unroll
        for (int k = 0; k < 1 + NS + NP; ++k)
          v[k] = lane_group_reduce<SumOp, kW>(k < 1 + NS ? pv[k] * f : pv[k]);
        r *= (mw == -INFINITY) ? 0.f : fast_exp2((mw - mm) * kLog2e);
        m = mm;
        this->phase ^= 1;
      }
    }
    o.max = m;
    o.sum = v[0];
    o.r = r;
#pragma unroll
    for (int k = 0; k < NS; ++k) o.scaled[k] = v[1 + k];
#pragma unroll
    for (int k = 0; k < NP; ++k) o.plain[k] = v[1 + NS + k];
    return o;
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
  // statistics of this thread's elements (two passes over registers: mean, then deviations)
  template <class A> __device__ __forceinline__ Welford local_welford(const A& val) const {
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
    return w;
  }
  // merge the threads' statistics over the team; every thread gets the row's
  __device__ __forceinline__ Welford xwelford(Welford w) {
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
  template <class A> __device__ __forceinline__ Welford welford(const A& val) { return xwelford(local_welford(val)); }
  // Online softmax of a row walked in chunks: the running (maximum, sum of exponentials
  // relative to it) of this thread absorbs one chunk; the team exchange follows the loop.
  struct MaxSum {
    float max, sum;
  };
  template <class A> __device__ __forceinline__ void online_chunk(MaxSum& acc, const A& val) const {
    float m = acc.max;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j)) m = fmaxf(m, Cast<float>::from(at(val, i * Base::kVec + j)));
    if (m == -INFINITY) return;      // nothing but -inf so far
    float s = acc.sum * fast_exp2((acc.max - m) * kLog2e);   // exp2(-inf) == 0 covers the first chunk
    const float shift = -m * kLog2e;
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
      for (int j = 0; j < Base::kVec; ++j)
        if (inside(i, j)) s += fast_exp2(fmaf(Cast<float>::from(at(val, i * Base::kVec + j)), kLog2e, shift));
    acc.max = m;
    acc.sum = s;
  }
  __device__ __forceinline__ MaxSum online_finish(MaxSum acc) {
    float m = acc.max, s[1] = {acc.sum}, none[1] = {0.f};
    if constexpr (TEAM < 32) {
      const float mw = lane_group_reduce<FastMaxOp, TEAM>(m);
      const float r = (m == -INFINITY) ? 0.f : fast_exp2((m - mw) * kLog2e);
      return MaxSum{mw, lane_group_reduce<SumOp, TEAM>(s[0] * r)};
    } else {
      Base::template reduce_rescaled<1, 0>(m, s, none, kLog2e);
      return MaxSum{m, s[0]};
    }
  }
  template <class A> __device__ __forceinline__ bool reduce_any(const A& val) {
    return reduce<MaxOp>(op::where(val, 1.f, 0.f)) != 0.f;
  }
};

// Per-column operand J of a generated body: the first KREGS operands (the most used ones) are
// registers of the thread, the others are read from the shared-memory table when needed.
template <int J, int KREGS, class Ctx, class U, int E>
__device__ __forceinline__ void kinit(Ctx& c, vf<E>& reg, const U* rowp) {
  if constexpr (J < KREGS) reg = c.load_row(rowp);
  else c.template fill_sconst<J - KREGS>(rowp);
}
template <int J, int KREGS, class Ctx, int E>
__device__ __forceinline__ vf<E> kget(const Ctx& c, const vf<E>& reg) {
  if constexpr (J < KREGS) return reg;
  else return c.template sconst<J - KREGS>();
}

// Order in which a row kernel with short rows walks its kept index.  The kept space is
// [A][LC][LB] with LB fastest (the order of the output), while the rows that are adjacent in
// memory are the ones that differ in the LC digit.  Walking it in TB x TC tiles - TC consecutive
// LC digits fastest, then TB consecutive LB digits - makes a warp read adjacent rows (one
// contiguous span) and lets the one-element-per-row results of a tile fill whole sectors, the
// job the reference gives its transposed tile (inductor_x/codegen/triton.py:856-888).
// B_FIRST: inside a tile the output digit runs fastest, so the rows a warp works on at once
// store one contiguous run (a full 32-byte sector for sixteen 16-bit results); chosen when a
// row is at least one 128-byte line, i.e. when reading rows that are far apart wastes nothing.
template <int LB, int LC, int TB, int TC, bool B_FIRST = false>
__device__ __forceinline__ long long tile_order(long long slot) {
  static_assert(LB % TB == 0 && LC % TC == 0, "tiles must divide both extents");
  constexpr long long kPlane = (long long)LB * LC;
  const long long a = slot / kPlane;
  const int rem = (int)(slot % kPlane);
  const int c_lo = B_FIRST ? (rem / TB) % TC : rem % TC;
  const int b_lo = B_FIRST ? rem % TB : (rem / TC) % TB;
  const int b_hi = (rem / (TC * TB)) % (LB / TB);
  const int c_hi = rem / (TC * LB);
  return a * kPlane + (long long)(c_hi * TC + c_lo) * LB + (b_hi * TB + b_lo);
}

// CTAs of a row kernel that fit on one SM, cached per device (the attribute is a property of
// the device the calling thread has current; several host threads may ask at once)
template <class K> inline int row_resident(K kern, int threads, size_t smem = 0) {
  static std::atomic<int> cache[64];
  int dev = 0;
  cudaGetDevice(&dev);
  const int slot = dev & 63;
  int n = cache[slot].load(std::memory_order_acquire);
  if (n == 0) {
    // static + dynamic shared memory beyond 48 KiB needs the opt-in, once per device
    if (smem > 32 * 1024 &&
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem) != cudaSuccess || n < 1) return -1;
    cache[slot].store(n, std::memory_order_release);
  }
  return n;
}

template <class Body, typename T, int TEAM, int TEAMS, int VPT, int MIN_CTAS, int PF, bool FULL, bool STAGED>
__global__ void __launch_bounds__(TEAM* TEAMS, MIN_CTAS)
    row_gen_kernel(const Body body, const long long rows, const int cols) {
  using Ctx = GenRowCtx<T, TEAM, TEAMS, VPT, FULL>;
  constexpr int kSlots = TEAM > 32 ? 2 * (TEAM / 32) * 4 : 1;  // exchange floats per team
  __shared__ __align__(16) float exchange[TEAMS * kSlots];
  extern __shared__ __align__(16) unsigned char operand_table[];   // Body::kSmemConsts slots
  Ctx c;
  c.lane = threadIdx.x % TEAM;
  c.team = threadIdx.x / TEAM;
  c.cols = cols;
  c.phase = 0;
  c.red = exchange + c.team * kSlots;
  c.ktab = reinterpret_cast<const float4*>(operand_table);
  // the next launch of the stream may place its CTAs as ours retire; no global access
  // happens before the launch ahead of us has completed
  pdl_launch_dependents();
  pdl_wait();
  const long long stride = (long long)gridDim.x * TEAMS;
  // the first row's vectors are requested before the per-column operands are loaded and
  // widened, so that both latencies overlap (it matters for kernels of a few microseconds)
  typename Body::Raw nxt;
  if constexpr (TEAM >= 32 && STAGED) {
    const long long r0 = (long long)blockIdx.x * TEAMS + c.team;
    if (r0 < rows) body.fetch(c, r0, nxt);
  }
  typename Body::Consts k;
  body.init(c, k);
  if constexpr (Body::kSmemConsts > 0) __syncthreads();   // the operand table is complete
  if constexpr (TEAM < 32) {
    // The teams of a warp run the same number of rows (full-mask shuffles inside).  Rows this
    // short give a thread one vector each, so kBatch rows are fetched before the first is
    // worked on: kBatch independent loads in flight per thread instead of one.
    constexpr int kBatch = STAGED ? 4 : 1;
    typename Body::Raw raw[kBatch];
    for (long long base = (long long)blockIdx.x * TEAMS; base < rows; base += stride * kBatch) {
      if constexpr (STAGED) {
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          const long long r = base + u * stride + c.team;
          body.fetch(c, r < rows ? r : rows - 1, raw[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const long long b = base + u * stride;
        if (b >= rows) break;            // uniform over the CTA
        const long long r = b + c.team;
        c.live = r < rows;
        body.template row<STAGED>(c, k, c.live ? r : rows - 1, raw[u]);
      }
    }
    return;
  } else {
    long long r = (long long)blockIdx.x * TEAMS + c.team;
    while (r < rows) {
      const typename Body::Raw cur = nxt;
      const long long rn = r + stride;
      if constexpr (STAGED) {
        if (rn < rows) body.fetch(c, rn, nxt);
      }
      // PF rows beyond the fetched one are on their way from DRAM to L2
      if constexpr (PF > 0) {
        const long long ahead = r + (PF + (STAGED ? 1 : 0)) * stride;
        if (ahead < rows) body.prefetch(c, ahead);
      }
      body.template row<STAGED>(c, k, r, cur);
      r = rn;
    }
  }
}
template <class Body, typename T, int TEAM, int TEAMS, int VPT, int MIN_CTAS = 1, int PF = 0, bool FULL = false>
int launch_row_gen(const Body& body, long long rows, int cols, void* stream, bool aligned = false) {
  if (rows <= 0) return 0;
  if (FULL && cols != TEAM * VPT * Elem<T>::kVec) return (int)cudaErrorInvalidValue;
  // a row longer than the team can hold (a run-time extent beyond the compiled capacity);
  // looped bodies walk any length in chunks
  if (cols < 0 || (!Body::kLooped && cols > TEAM * VPT * Elem<T>::kVec)) return (int)cudaErrorInvalidValue;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long groups = (rows + TEAMS - 1) / TEAMS;
  using Ctx = GenRowCtx<T, TEAM, TEAMS, VPT, FULL>;
  const size_t smem = (size_t)Body::kSmemConsts * Ctx::kQuads * Ctx::kTabVecs * sizeof(float4);
  if (aligned) {
    auto kern = row_gen_kernel<Body, T, TEAM, TEAMS, VPT, MIN_CTAS, PF, FULL, true>;
    const int resident = row_resident(kern, TEAM * TEAMS, smem);
    if (resident < 1) return (int)cudaErrorInvalidConfiguration;
    long long grid = (long long)sms * resident;
    if (grid > groups) grid = groups;
    return (int)launch_pdl(kern, (unsigned)grid, TEAM * TEAMS, smem, (cudaStream_t)stream, body, rows, cols);
  }
  auto kern = row_gen_kernel<Body, T, TEAM, TEAMS, VPT, MIN_CTAS, PF, FULL, false>;
  const int resident = row_resident(kern, TEAM * TEAMS, smem);
  if (resident < 1) return (int)cudaErrorInvalidConfiguration;
  long long grid = (long long)sms * resident;
  if (grid > groups) grid = groups;
  return (int)launch_pdl(kern, (unsigned)grid, TEAM * TEAMS, smem, (cudaStream_t)stream, body, rows, cols);
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
  // the reduced indices this thread row walks, and who stores the result of a tile
  __device__ __forceinline__ long long rbegin() const { return ty; }
  __device__ __forceinline__ long long rstep() const { return TY; }
  __device__ __forceinline__ bool writer() const { return ty == 0; }

  template <int N> static __device__ __forceinline__ vf<N> splat(float v) {
    vf<N> r;
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = v;
    return r;
  }
  using ISum = ::ixb::gen::ISum;
  using IProd = ::ixb::gen::IProd;
  using IMax = ::ixb::gen::IMax;
  using IMin = ::ixb::gen::IMin;
  template <int N> static __device__ __forceinline__ vi<N> splat_int(long long v) {
    vi<N> r;
#pragma unroll
    for (int i = 0; i < N; ++i) r.v[i] = v;
    return r;
  }
  // exact integer fold: the shared scratch is sized for floats, so the 64-bit partials of
  // the warps cross it in two rounds (low and high halves would not fold; values do)
  template <class IOp> __device__ __forceinline__ vi<V> combine_int(const vi<V>& acc) {
    vi<V> r = acc;
#pragma unroll
    for (int off = TX; off < 32; off <<= 1)
#pragma unroll
      for (int i = 0; i < V; ++i) r.v[i] = IOp::f(r.v[i], __shfl_xor_sync(kFull, r.v[i], off));
    if constexpr (kWarps > 1) {
      const int warp = (ty * TX + tx) >> 5;
      long long* ipart = reinterpret_cast<long long*>(part);
      // the scratch holds kWarps * TX * V floats = half as many 64-bit values: fold the
      // vector in two halves
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        constexpr int HV = (V + 1) / 2;
        if (ty % kRowsPerWarp == 0) {
#pragma unroll
          for (int i = 0; i < HV; ++i)
            if (h * HV + i < V) ipart[(warp * TX + tx) * HV + i] = r.v[h * HV + i];
        }
        __syncthreads();
        if (writer()) {
#pragma unroll
          for (int i = 0; i < HV; ++i) {
            if (h * HV + i < V) {
              long long a = ipart[tx * HV + i];
#pragma unroll
              for (int w = 1; w < kWarps; ++w) a = IOp::f(a, ipart[(w * TX + tx) * HV + i]);
              r.v[h * HV + i] = a;
            }
          }
        }
        __syncthreads();
      }
    }
    return r;
  }
  // fold the TY partial vectors; the writer row receives the result
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
      // only the thread row that stores the tile needs the folded vector (a generated outer
      // kernel has one reduction and nothing after it but the store): the other rows skip
      // the kWarps x V shared-memory reads
      if (writer()) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          float a = part[tx * V + i];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) a = Op::combine(a, part[(w * TX + tx) * V + i]);
          r.v[i] = a;
        }
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
// ---- outer reduction split over a thread-block cluster -----------------------------------------
// When the kept extent gives fewer tiles than the GPU has SMs and the reduced axis is long, a
// cluster of CS CTAs shares one tile: rank k walks the reduced indices k * TY + ty, + TY * CS, ...
// and the partial vectors meet in the shared memory of rank 0 (distributed shared memory):
// every other rank stores its vector there (st.shared::cluster to the address mapa gives) and
// arrives on rank 0's mbarrier with cluster-scope release; rank 0 waits on it with a bounded
// acquire wait, folds and stores.  This is the reference's outer split
// (inductor_x/codegen/split_tiling.py:159-165), which combines with atomic adds in global
// memory; here nothing leaves the chip.  One tile per cluster, so the inbox is used once.
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_rank(const void* local_smem, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_smem)), "r"(rank));
  return remote;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
// bounded wait with cluster-scope acquire (the data was written by other CTAs of the cluster)
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  const long long t0 = clock64();
  while (true) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, 1000000;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
    if (clock64() - t0 > kWaitCycles) {
      atomicAdd(&g_wait_timeouts, 1u);
      return false;
    }
  }
}

template <int V, int TX, int TY, int CS> struct OuterSplitCtx : OuterCtx<V, TX, TY> {
  using Base = OuterCtx<V, TX, TY>;
  int rank = 0;      // CTA rank inside the cluster
  float* inbox;      // [CS - 1][TX * V]; only rank 0's copy is written to
  uint64_t* bar;     // arrivals of the other ranks; only rank 0's copy is used
  bool ok = true;    // false after rank 0's wait gave up: the tile is not stored
  __device__ __forceinline__ long long rbegin() const { return (long long)rank * TY + this->ty; }
  __device__ __forceinline__ long long rstep() const { return (long long)TY * CS; }
  __device__ __forceinline__ bool writer() const { return this->ty == 0 && rank == 0 && ok; }
  template <class Op> __device__ __forceinline__ vf<V> combine(const vf<V>& acc) {
    vf<V> r = Base::template combine<Op>(acc);   // the CTA's own partial, in every thread row
    if (this->ty != 0) return r;
    if (rank != 0) {
      const uint32_t dst = map_to_rank(inbox + ((rank - 1) * TX + this->tx) * V, 0);
#pragma unroll
      for (int i = 0; i < V; ++i) st_cluster_f32(dst + 4 * i, r.v[i]);
      mbar_arrive_remote(map_to_rank(bar, 0));
    } else {
      ok = mbar_wait_cluster(bar, 0);
      if (ok) {
#pragma unroll
        for (int k = 0; k < CS - 1; ++k)
#pragma unroll
          for (int i = 0; i < V; ++i) r.v[i] = Op::combine(r.v[i], inbox[(k * TX + this->tx) * V + i]);
      }
    }
    return r;
  }
};

template <class Body, int TX, int TY, int CS, bool ALIGNED>
__global__ void __launch_bounds__(TX* TY) outer_split_gen_kernel(const Body body, const long long xnumel) {
  constexpr int V = Body::kVec;
  __shared__ __align__(16) float part[(TX * TY / 32) * TX * V];
  __shared__ __align__(16) float inbox[(CS - 1) * TX * V];
  __shared__ __align__(8) uint64_t bar;
  OuterSplitCtx<V, TX, TY, CS> c;
  c.tx = threadIdx.x % TX;
  c.ty = threadIdx.x / TX;
  c.part = part;
  c.inbox = inbox;
  c.bar = &bar;
  c.rank = (int)cluster_rank();
  if (c.rank == 0 && threadIdx.x == 0) {
    mbar_init(&bar, (CS - 1) * TX);
    mbar_init_fence();
  }
  // every CTA of the cluster is resident and rank 0's barrier is initialised before anyone pushes
  cluster_sync_all();
  const long long per_cta = (long long)TX * V;
  const long long t = blockIdx.x / CS;   // one tile per cluster
  const long long xbase = t * per_cta + (long long)c.tx * V;
  const long long left = xnumel - xbase;
  if (ALIGNED && xnumel - t * per_cta >= per_cta) body.template tile<true>(c, xbase, V);
  else body.template tile<false>(c, xbase, left >= V ? V : (left > 0 ? (int)left : 0));
}
template <class Body, int TX, int CS>
int launch_outer_split_gen(const Body& body, long long xnumel, void* stream, bool aligned = false) {
  if (xnumel <= 0) return 0;
  constexpr int TY = 256 / TX;
  const long long per_cta = (long long)TX * Body::kVec;
  const long long tiles = (xnumel + per_cta - 1) / per_cta;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * CS));
  cfg.blockDim = dim3(TX * TY);
  cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (aligned) return (int)cudaLaunchKernelEx(&cfg, outer_split_gen_kernel<Body, TX, TY, CS, true>, body, xnumel);
  return (int)cudaLaunchKernelEx(&cfg, outer_split_gen_kernel<Body, TX, TY, CS, false>, body, xnumel);
}

template <class Body, int TX = 32>
int launch_outer_gen(const Body& body, long long xnumel, void* stream, bool aligned = false) {
  if (xnumel <= 0) return 0;
  constexpr int TY = 256 / TX;
  static const long long cap_a = resident_ctas(outer_gen_kernel<Body, TX, TY, true>, TX * TY);
  static const long long cap_u = resident_ctas(outer_gen_kernel<Body, TX, TY, false>, TX * TY);
  const long long per_cta = (long long)TX * Body::kVec;
  long long grid = (xnumel + per_cta - 1) / per_cta;
  // A tile ends with a CTA-wide fold during which the CTA has no loads in flight, so the grid
  // holds several waves of CTAs (the hardware starts the next CTA's loads while another folds)
  // instead of exactly the resident set.  IXB_OUTER_WAVES overrides the default.
  static const long long waves = [] {
    const char* v = getenv("IXB_OUTER_WAVES");
    const long long w = v != nullptr ? atoll(v) : 2;
    return w < 1 ? 1 : w;
  }();
  const long long cap = (aligned ? cap_a : cap_u) * waves;
  if (grid > cap) grid = cap;
  if (aligned) outer_gen_kernel<Body, TX, TY, true><<<(unsigned)grid, TX * TY, 0, (cudaStream_t)stream>>>(body, xnumel);
  else outer_gen_kernel<Body, TX, TY, false><<<(unsigned)grid, TX * TY, 0, (cudaStream_t)stream>>>(body, xnumel);
  return (int)cudaGetLastError();
}

}  // namespace gen
}  // namespace ixb
