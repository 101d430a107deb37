// Pre-instantiated bodies for the persistent row template (row.cuh).  Each body is the
// fused math of one graph the backend meets on its hot path; generated functor modules
// define bodies of the same shape for everything else.
#pragma once
#include "row.cuh"

namespace ixb {

// -------------------------------------------------------------------------------------
// out[r] = sum_c gelu(x[r,c] * w[c] + b[c])          (fp32, erf GELU)
// The reference cannot fuse this graph: gelu has neither a decomposition nor a fusable
// lowering there (inductor_x/decomposition.py:8-25, inductor_x/lowering.py:185-198), so
// it runs mul+add, an extern gelu and a sum as three kernels.  Here it is one pass.
// -------------------------------------------------------------------------------------
struct AffineGeluRowSum {
  using in_t = float;
  static constexpr int kRowInputs = 1;
  struct Params {
    const float* x;
    const float* w;
    const float* b;
    float* out;
  };
  static __device__ __forceinline__ const float* row_ptr(const Params& p, int) { return p.x; }

  template <int VPT> struct Impl {
    // per-column constants stay in registers while the footprint is small, otherwise
    // they are re-read through L1 (8 KiB in total, always resident)
    static constexpr bool kCache = VPT <= 2;
    float w_[kCache ? VPT : 1][4], b_[kCache ? VPT : 1][4];

    template <class Ctx> __device__ __forceinline__ void init(const Params& p, const Ctx& c) {
      if constexpr (kCache) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          unpack<float>(c.template load<false>(p.w, i), w_[i]);
          unpack<float>(c.template load<false>(p.b, i), b_[i]);
        }
      }
    }
    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[1][VPT]) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float x[4], w[4], b[4];
        unpack<float>(raw[0][i], x);
        if constexpr (kCache) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            w[j] = w_[i][j];
            b[j] = b_[i][j];
          }
        } else {
          unpack<float>(c.template load<false>(p.w, i), w);
          unpack<float>(c.template load<false>(p.b, i), b);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (c.ok(i, j)) acc += gelu_erf(fmaf(x[j], w[j], b[j]));
      }
      acc = c.template reduce<SumOp>(acc);
      if (c.lane == 0) p.out[r] = acc;
    }
  };
};

// -------------------------------------------------------------------------------------
// y = layer_norm(softmax(x, -1) * g + x, gamma, beta, eps)   over the last axis.
// Four reductions (row max, sum of exponentials, mean, centred second moment) run on
// registers; the variance is the two-pass form the reference lowers var_mean to
// (inductor_x/lowering.py:270-325).  All arithmetic is fp32; only x, g, gamma, beta and
// y are stored in the half type.
// -------------------------------------------------------------------------------------
template <typename T> struct SoftmaxLayerNorm {
  using in_t = T;
  static constexpr int kRowInputs = 1;
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    const T* g;
    const T* gamma;
    const T* beta;
    T* y;
    float eps;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }

  template <int VPT> struct Impl {
    uint4 g_[VPT], gamma_[VPT], beta_[VPT];  // packed per-column constants

    template <class Ctx> __device__ __forceinline__ void init(const Params& p, const Ctx& c) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        g_[i] = c.template load<false>(p.g, i);
        gamma_[i] = c.template load<false>(p.gamma, i);
        beta_[i] = c.template load<false>(p.beta, i);
      }
    }
    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[1][VPT]) {
      float x[VPT][kVec], e[VPT][kVec];
      float m = -INFINITY;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        unpack<T>(raw[0][i], x[i]);
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          if (c.ok(i, j)) m = fmaxf(m, x[i][j]);
      }
      m = c.template reduce<FastMaxOp>(m);
      const float ml = m * kLog2e;
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          e[i][j] = c.ok(i, j) ? exp2f(fmaf(x[i][j], kLog2e, -ml)) : 0.f;
          s += e[i][j];
        }
      }
      s = c.template reduce<SumOp>(s);
      const float inv = 1.f / s;
      float tsum = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float g[kVec];
        unpack<T>(g_[i], g);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          x[i][j] = c.ok(i, j) ? fmaf(e[i][j] * inv, g[j], x[i][j]) : 0.f;
          tsum += x[i][j];
        }
      }
      const float inv_n = 1.f / (float)c.cols;
      const float mean = c.template reduce<SumOp>(tsum) * inv_n;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          x[i][j] = c.ok(i, j) ? x[i][j] - mean : 0.f;
          q = fmaf(x[i][j], x[i][j], q);
        }
      }
      const float var = c.template reduce<SumOp>(q) * inv_n;
      const float rstd = rsqrtf(var + p.eps);
      T* yrow = p.y + r * (long long)c.cols;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float ga[kVec], be[kVec], y[kVec];
        unpack<T>(gamma_[i], ga);
        unpack<T>(beta_[i], be);
#pragma unroll
        for (int j = 0; j < kVec; ++j) y[j] = fmaf(x[i][j] * rstd, ga[j], be[j]);
        c.store(yrow, i, y);
      }
    }
  };
};

// -------------------------------------------------------------------------------------
// RMSNorm with an optional fused residual add (Llama-style decoder layer):
//   h = x (+ res);  y = h * rsqrt(mean(h^2) + eps) * w;  optionally h is written too.
// -------------------------------------------------------------------------------------
template <typename T, bool RESIDUAL> struct RmsNorm {
  using in_t = T;
  static constexpr int kRowInputs = RESIDUAL ? 2 : 1;
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    const T* res;    // RESIDUAL only
    const T* w;
    T* y;
    T* h_out;        // RESIDUAL only; may be null
    float eps;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int k) {
    return k == 0 ? p.x : p.res;
  }
  template <int VPT> struct Impl {
    uint4 w_[VPT];
    template <class Ctx> __device__ __forceinline__ void init(const Params& p, const Ctx& c) {
#pragma unroll
      for (int i = 0; i < VPT; ++i)
        w_[i] = c.template load<false>(p.w, i);
    }
    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[kRowInputs][VPT]) {
      float h[VPT][kVec];
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        unpack<T>(raw[0][i], h[i]);
        if constexpr (RESIDUAL) {
          float rr[kVec];
          unpack<T>(raw[kRowInputs - 1][i], rr);
          // the sum is rounded to the storage type first: it is the tensor the next
          // layer reads, and eager PyTorch normalises exactly that rounded value
#pragma unroll
          for (int j = 0; j < kVec; ++j) h[i][j] = Elem<T>::to_f(Elem<T>::from_f(h[i][j] + rr[j]));
          if (p.h_out != nullptr) c.store(p.h_out + r * (long long)c.cols, i, h[i]);
        }
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          if (c.ok(i, j)) q = fmaf(h[i][j], h[i][j], q);
      }
      q = c.template reduce<SumOp>(q);
      const float rstd = rsqrtf(q / (float)c.cols + p.eps);
      T* yrow = p.y + r * (long long)c.cols;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float w[kVec], y[kVec];
        unpack<T>(w_[i], w);
#pragma unroll
        for (int j = 0; j < kVec; ++j) y[j] = h[i][j] * rstd * w[j];
        c.store(yrow, i, y);
      }
    }
  };
};

// -------------------------------------------------------------------------------------
// Plain reductions of the last axis: sum, mean, amax, amin, prod, and the two-pass
// var_mean the reference uses.  One value (or two) per row.
// -------------------------------------------------------------------------------------
enum RowReduceKind { kRowSum = 0, kRowMean = 1, kRowAmax = 2, kRowAmin = 3, kRowProd = 4 };

template <typename T, int KIND> struct RowReduce {
  using in_t = T;
  static constexpr int kRowInputs = 1;
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    T* out;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }
  using Op = typename std::conditional<
      KIND == kRowAmax, MaxOp,
      typename std::conditional<KIND == kRowAmin, MinOp,
                                typename std::conditional<KIND == kRowProd, ProdOp, SumOp>::type>::type>::type;
  template <int VPT> struct Impl {
    template <class Ctx> __device__ __forceinline__ void init(const Params&, const Ctx&) {}
    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[1][VPT]) {
      float acc = Op::identity();
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float x[kVec];
        unpack<T>(raw[0][i], x);
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          if (c.ok(i, j)) acc = Op::combine(acc, x[j]);
      }
      acc = c.template reduce<Op>(acc);
      if constexpr (KIND == kRowMean) acc /= (float)c.cols;
      if (c.lane == 0) p.out[r] = Elem<T>::from_f(acc);
    }
  };
};

// var_mean over the last axis: mean first, then the centred sum of squares
// (inductor_x/lowering.py:270-325 disables Welford in favour of this two-pass form).
template <typename T> struct RowVarMean {
  using in_t = T;
  static constexpr int kRowInputs = 1;
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    T* var;
    T* mean;
    float correction;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }
  template <int VPT> struct Impl {
    template <class Ctx> __device__ __forceinline__ void init(const Params&, const Ctx&) {}
    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[1][VPT]) {
      float x[VPT][kVec];
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        unpack<T>(raw[0][i], x[i]);
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          if (c.ok(i, j)) s += x[i][j];
      }
      const float mean = c.template reduce<SumOp>(s) / (float)c.cols;
      float q = 0.f;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          const float d = c.ok(i, j) ? x[i][j] - mean : 0.f;
          q = fmaf(d, d, q);
        }
      }
      q = c.template reduce<SumOp>(q);
      if (c.lane == 0) {
        p.var[r] = Elem<T>::from_f(q / fmaxf((float)c.cols - p.correction, 0.f));
        p.mean[r] = Elem<T>::from_f(mean);
      }
    }
  };
};

// argmax / argmin over the last axis (int64 result, first occurrence wins).
template <typename T, bool IS_MAX> struct RowArg {
  using in_t = T;
  static constexpr int kRowInputs = 1;
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    long long* out;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }
  template <int VPT> struct Impl {
    template <class Ctx> __device__ __forceinline__ void init(const Params&, const Ctx&) {}
    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[1][VPT]) {
      ArgPair best = ArgOp<IS_MAX>::identity();
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        float x[kVec];
        unpack<T>(raw[0][i], x);
#pragma unroll
        for (int j = 0; j < kVec; ++j)
          if (c.ok(i, j))
            best = ArgOp<IS_MAX>::combine(best, ArgPair{x[j], (long long)(c.vec_col(i) + j)});
      }
      best = c.template reduce_arg<IS_MAX>(best);
      if (c.lane == 0) p.out[r] = best.i;
    }
  };
};

}  // namespace ixb
