// Device-side building blocks shared by every kernel template of the B200 backend:
// 128-bit vector access, dtype packing, warp / team reductions and the math used by
// the pre-instantiated functors.  Header-only so that generated functor modules can
// include the same code as the prebuilt library.
#pragma once
#include <cstdlib>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <float.h>

namespace ixb {

using bf16 = __nv_bfloat16;
using f16 = __half;

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// ---------------------------------------------------------------------------------
// Element traits: how many elements one 128-bit vector holds and how to widen /
// narrow them.  Half types are always computed in fp32 (the reference upcasts every
// half load, inductor_x/codegen/triton.py:1431-1433).
// ---------------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kVec = 4;
  static __device__ __forceinline__ float to_f(float v) { return v; }
  static __device__ __forceinline__ float from_f(float v) { return v; }
};
template <> struct Elem<f16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_f(f16 v) { return __half2float(v); }
  static __device__ __forceinline__ f16 from_f(float v) { return __float2half_rn(v); }
};
template <> struct Elem<bf16> {
  static constexpr int kVec = 8;
  static __device__ __forceinline__ float to_f(bf16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ bf16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Layout-only element type: KV elements per thread vector, for rows of a storage type the
// prebuilt bodies never load themselves (integers, booleans); generated bodies bring their
// own typed loads and use the row context only for the column arithmetic.
template <int KV> struct Lanes {};
template <int KV> struct Elem<Lanes<KV>> {
  static constexpr int kVec = KV;
};

// 128-bit global access.  Inputs that are read once stream through L1 without
// allocating; outputs use a streaming store so they do not evict reusable lines.
__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ uint4 ldg_keep(const void* p) {
  return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void stg_stream(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Widen one 128-bit vector into fp32 lanes.
template <typename T> __device__ __forceinline__ void unpack(const uint4& raw, float* out);
template <> __device__ __forceinline__ void unpack<float>(const uint4& raw, float* out) {
  out[0] = __uint_as_float(raw.x);
  out[1] = __uint_as_float(raw.y);
  out[2] = __uint_as_float(raw.z);
  out[3] = __uint_as_float(raw.w);
}
template <> __device__ __forceinline__ void unpack<bf16>(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void unpack<f16>(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}

// Narrow fp32 lanes into one 128-bit vector (round to nearest even).
template <typename T> __device__ __forceinline__ uint4 pack(const float* in);
template <> __device__ __forceinline__ uint4 pack<float>(const float* in) {
  return make_uint4(__float_as_uint(in[0]), __float_as_uint(in[1]), __float_as_uint(in[2]),
                    __float_as_uint(in[3]));
}
template <> __device__ __forceinline__ uint4 pack<bf16>(const float* in) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}
template <> __device__ __forceinline__ uint4 pack<f16>(const float* in) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2 h = __floats2half2_rn(in[2 * i], in[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&h);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---------------------------------------------------------------------------------
// Reduction operators.  `combine` must be associative and commutative.
// ---------------------------------------------------------------------------------
struct SumOp {
  static __device__ __forceinline__ float identity() { return 0.f; }
  static __device__ __forceinline__ float combine(float a, float b) { return a + b; }
};
// max / min propagate NaN like torch.amax / torch.amin.
struct MaxOp {
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  static __device__ __forceinline__ float combine(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
};
struct MinOp {
  static __device__ __forceinline__ float identity() { return INFINITY; }
  static __device__ __forceinline__ float combine(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
  }
};
// Non-propagating max for values known to be finite (softmax row maximum).
struct FastMaxOp {
  static __device__ __forceinline__ float identity() { return -INFINITY; }
  static __device__ __forceinline__ float combine(float a, float b) { return fmaxf(a, b); }
};
struct ProdOp {
  static __device__ __forceinline__ float identity() { return 1.f; }
  static __device__ __forceinline__ float combine(float a, float b) { return a * b; }
};

template <class Op> __device__ __forceinline__ float warp_reduce(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::combine(v, __shfl_xor_sync(kFull, v, o));
  return v;
}
// Reduce within aligned groups of WIDTH lanes (WIDTH a power of two <= 32).
template <class Op, int WIDTH> __device__ __forceinline__ float lane_group_reduce(float v) {
#pragma unroll
  for (int o = WIDTH / 2; o > 0; o >>= 1) v = Op::combine(v, __shfl_xor_sync(kFull, v, o));
  return v;
}

// (value, index) pair for arg-reductions.  Ties resolve to the smaller index and a NaN
// value wins over any number, matching torch.argmax / torch.argmin.
struct ArgPair {
  float v;
  long long i;
};
template <bool IS_MAX> struct ArgOp {
  static __device__ __forceinline__ ArgPair identity() {
    return ArgPair{IS_MAX ? -INFINITY : INFINITY, 0x7fffffffffffffffLL};
  }
  static __device__ __forceinline__ ArgPair combine(ArgPair a, ArgPair b) {
    const bool a_nan = a.v != a.v, b_nan = b.v != b.v;
    bool take_b;
    if (a_nan || b_nan) {
      take_b = b_nan && (!a_nan || b.i < a.i);
    } else if (a.v == b.v) {
      take_b = b.i < a.i;
    } else {
      take_b = IS_MAX ? (b.v > a.v) : (b.v < a.v);
    }
    return take_b ? b : a;
  }
};
template <bool IS_MAX> __device__ __forceinline__ ArgPair warp_reduce_arg(ArgPair p) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair q;
    q.v = __shfl_xor_sync(kFull, p.v, o);
    q.i = __shfl_xor_sync(kFull, p.i, o);
    p = ArgOp<IS_MAX>::combine(p, q);
  }
  return p;
}

// Warp-wide maximum in one instruction (sm_100a redux on fp32).
__device__ __forceinline__ float warp_max_fast(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}
// Three-input maximum (one instruction on sm_100).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// ---- programmatic dependent launch ----------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with programmatic stream serialization allowed: a kernel that calls pdl_wait()
// before its first global access may be scheduled while the previous kernel of the stream
// drains.  IXB_PDL=0 in the environment turns the attribute off.
inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("IXB_PDL");
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}
template <class K, class... Args>
inline cudaError_t launch_pdl(K kern, unsigned grid, unsigned block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Named barrier over `nthreads` threads (a multiple of 32); id 0 is __syncthreads().
__device__ __forceinline__ void team_barrier(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------
// Math used by the pre-instantiated functors.
// ---------------------------------------------------------------------------------
// exact-erf GELU, the default of torch.nn.functional.gelu.
__device__ __forceinline__ float gelu_erf(float v) {
  return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f));
}
// exact-erf GELU without erff: gelu(v) = relu(v) - |v| * Phi(-|v|) and
// Phi(-a) = 2^-G(a), with G fitted by a degree-6 polynomial on [0, 6] (weighted so that
// the error of the product is uniform).  Max abs error against the fp64 erf form over
// [-8, 8] is 2.8e-7 - below fp32 rounding of the terms it is summed with - for about
// half the instructions of erff.  Beyond |v| = 12 the correction term is < 2^-90 and the
// argument is clamped so the polynomial is never extrapolated.
__device__ __forceinline__ float gelu_erf_fast(float v) {
  const float a = fabsf(v);
  const float t = fminf(a, 12.f);
  float g = -3.309498788439669e-05f;
  g = fmaf(g, t, 0.0007692387443967164f);
  g = fmaf(g, t, -0.008080779574811459f);
  g = fmaf(g, t, 0.05341219902038574f);
  g = fmaf(g, t, 0.45877090096473694f);
  g = fmaf(g, t, 1.1512017250061035f);
  g = fmaf(g, t, 0.999993085861206f);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-g));
  return fmaf(-a, e, fmaxf(v, 0.f));
}
__device__ __forceinline__ float fast_exp2(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

constexpr float kLog2e = 1.4426950408889634f;

// Packed fp32x2 arithmetic (one issue slot for two lanes on sm_100).
#ifdef IXB_SCALAR_PAIRS
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  return make_float2(fmaf(a.x, b.x, c.x), fmaf(a.y, b.y, c.y));
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return make_float2(a.x * b.x, a.y * b.y); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
#else
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<const unsigned long long*>(&a)),
        "l"(*reinterpret_cast<const unsigned long long*>(&b)),
        "l"(*reinterpret_cast<const unsigned long long*>(&c)));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<const unsigned long long*>(&a)),
        "l"(*reinterpret_cast<const unsigned long long*>(&b)));
  return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  float2 d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<const unsigned long long*>(&a)),
        "l"(*reinterpret_cast<const unsigned long long*>(&b)));
  return d;
}
#endif

// gelu_erf_fast on two values: same operations, the polynomial on packed pairs.
__device__ __forceinline__ float2 gelu_erf_fast2(float2 v) {
  const float2 a = make_float2(fabsf(v.x), fabsf(v.y));
  const float2 t = make_float2(fminf(a.x, 12.f), fminf(a.y, 12.f));
  // coefficients negated: the polynomial yields -g, the argument of the exponential
  float2 g = fma2(make_float2(3.309498788439669e-05f, 3.309498788439669e-05f), t,
                  make_float2(-0.0007692387443967164f, -0.0007692387443967164f));
  g = fma2(g, t, make_float2(0.008080779574811459f, 0.008080779574811459f));
  g = fma2(g, t, make_float2(-0.05341219902038574f, -0.05341219902038574f));
  g = fma2(g, t, make_float2(-0.45877090096473694f, -0.45877090096473694f));
  g = fma2(g, t, make_float2(-1.1512017250061035f, -1.1512017250061035f));
  g = fma2(g, t, make_float2(-0.999993085861206f, -0.999993085861206f));
  float ex, ey;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"(g.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ey) : "f"(g.y));
  return make_float2(fmaf(-a.x, ex, fmaxf(v.x, 0.f)), fmaf(-a.y, ey, fmaxf(v.y, 0.f)));
}

}  // namespace ixb
