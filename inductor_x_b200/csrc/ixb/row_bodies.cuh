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
  static __host__ __device__ constexpr size_t smem_bytes(int, int) { return 0; }
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

    template <class Ctx>
    __device__ __forceinline__ void init(const Params& p, const Ctx& c, unsigned char*) {
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
      float2 acc2 = make_float2(0.f, 0.f);
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
        if constexpr (Ctx::kAligned) {
          // whole vectors are valid or not: two elements per issue slot through the affine
          // step and the polynomial of the GELU
          if (c.valid(i)) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
              const float2 v = fma2(make_float2(x[j], x[j + 1]), make_float2(w[j], w[j + 1]),
                                    make_float2(b[j], b[j + 1]));
              acc2 = add2(acc2, gelu_erf_fast2(v));
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (c.ok(i, j)) acc += gelu_erf_fast(fmaf(x[j], w[j], b[j]));
        }
      }
      acc += acc2.x + acc2.y;
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
template <typename T, int WIDE_VPT = 2> struct SoftmaxLayerNorm {
  using in_t = T;
  static constexpr int kRowInputs = 1;
  static constexpr int kVec = Elem<T>::kVec;
  static constexpr int H = kVec / 2;       // fp32 pairs per vector
  static constexpr int kQuads = kVec / 4;  // float4 groups per vector
  struct Params {
    const T* x;
    const T* g;
    const T* gamma;
    const T* beta;
    T* y;
    float eps;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }
  // With more than two vectors per thread the widened per-column constants no longer fit
  // in registers; they live in shared memory as fp32, laid out [array][quad][vector][4]
  // so that consecutive lanes read consecutive 16-byte words (no bank conflicts).
  static __host__ __device__ constexpr size_t smem_bytes(int cols, int vpt) {
    return vpt <= WIDE_VPT ? 0 : (size_t)3 * kQuads * ((cols + kVec - 1) / kVec) * 16;
  }

  template <int VPT> struct Impl {
    static constexpr bool kWide = VPT <= WIDE_VPT;
    float2 gw_[kWide ? VPT : 1][H], gaw_[kWide ? VPT : 1][H], bew_[kWide ? VPT : 1][H];
    const float4* tab_;  // shared-memory table (VPT > 2)
    int nvec_;

    template <class Ctx>
    __device__ __forceinline__ void init(const Params& p, const Ctx& c, unsigned char* smem) {
      if constexpr (kWide) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          unpack<T>(c.template load<false>(p.g, i), reinterpret_cast<float*>(gw_[i]));
          unpack<T>(c.template load<false>(p.gamma, i), reinterpret_cast<float*>(gaw_[i]));
          unpack<T>(c.template load<false>(p.beta, i), reinterpret_cast<float*>(bew_[i]));
        }
      } else {
        nvec_ = (c.cols + kVec - 1) / kVec;
        float4* tab = reinterpret_cast<float4*>(smem);
        tab_ = tab;
        const T* src[3] = {p.g, p.gamma, p.beta};
        for (int v = threadIdx.x; v < nvec_; v += blockDim.x) {
#pragma unroll
          for (int a = 0; a < 3; ++a) {
            float f[kVec];
#pragma unroll
            for (int j = 0; j < kVec; ++j)
              f[j] = (v * kVec + j < c.cols) ? Elem<T>::to_f(src[a][v * kVec + j]) : 0.f;
#pragma unroll
            for (int qd = 0; qd < kQuads; ++qd)
              tab[(a * kQuads + qd) * nvec_ + v] =
                  make_float4(f[4 * qd], f[4 * qd + 1], f[4 * qd + 2], f[4 * qd + 3]);
          }
        }
        __syncthreads();
      }
    }

    // constants of array `a` (0 g, 1 gamma, 2 beta) for vector i of this thread
    template <class Ctx>
    __device__ __forceinline__ void constants(const Ctx& c, int a, int i, float2 (&out)[H]) const {
      if constexpr (kWide) {
#pragma unroll
        for (int h = 0; h < H; ++h) out[h] = a == 0 ? gw_[i][h] : (a == 1 ? gaw_[i][h] : bew_[i][h]);
      } else {
        const int v = c.lane + i * Ctx::kTeam;
#pragma unroll
        for (int qd = 0; qd < kQuads; ++qd) {
          // vectors past the end of the row have no table entry
          const float4 q4 = v < nvec_ ? tab_[(a * kQuads + qd) * nvec_ + v]
                                      : make_float4(0.f, 0.f, 0.f, 0.f);
          out[2 * qd] = make_float2(q4.x, q4.y);
          out[2 * qd + 1] = make_float2(q4.z, q4.w);
        }
      }
    }

    template <class Ctx>
    __device__ __forceinline__ void row(const Params& p, Ctx& c, long long r,
                                        const uint4 (&raw)[1][VPT]) {
      if constexpr (Ctx::kAligned) {
        row_packed(p, c, r, raw);
      } else {
        row_scalar(p, c, r, raw);
      }
    }

    // Aligned rows: validity is per vector and the element math runs on fp32 pairs
    // (fma/mul/add.f32x2: one issue slot per two elements).  Two exchanges per row.
    template <class Ctx>
    __device__ __forceinline__ void row_packed(const Params& p, Ctx& c, long long r,
                                               const uint4 (&raw)[1][VPT]) {
      // Pass A: widen, thread-local maximum and sum of x.
      float2 x[VPT][H], e[VPT][H];
      float m = -INFINITY;
      float2 sx2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        unpack<T>(raw[0][i], reinterpret_cast<float*>(x[i]));
        if (c.valid(i)) {
#pragma unroll
          for (int h = 0; h < H; ++h) {
            m = max3(m, x[i][h].x, x[i][h].y);
            sx2 = add2(sx2, x[i][h]);
          }
        }
      }
      // Pass B: exponentials relative to the thread's own maximum, their sum and their
      // g-weighted sum (online softmax: one exchange instead of max-then-sum).
      const float2 l2 = make_float2(kLog2e, kLog2e);
      const float2 nml = make_float2(-m * kLog2e, -m * kLog2e);
      float2 s2 = make_float2(0.f, 0.f), sg2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        if (c.valid(i)) {
          float2 g[H];
          constants(c, 0, i, g);
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const float2 a = fma2(x[i][h], l2, nml);
            e[i][h] = make_float2(fast_exp2(a.x), fast_exp2(a.y));
            s2 = add2(s2, e[i][h]);
            sg2 = fma2(e[i][h], g[h], sg2);
          }
        }
      }
      float sums[2] = {s2.x + s2.y, sg2.x + sg2.y};
      float sxa[1] = {sx2.x + sx2.y};
      const float rt = c.template reduce_rescaled<2, 1>(m, sums, sxa, kLog2e);
      const float inv = 1.f / sums[0];
      const float inv_n = 1.f / (float)c.cols;
      // mean(softmax*g + x) = (sum(e*g)/sum(e) + sum(x)) / n, by linearity
      const float mean = fmaf(sums[1], inv, sxa[0]) * inv_n;
      const float f = rt * inv;
      const float2 f2 = make_float2(f, f);
      const float2 nmean = make_float2(-mean, -mean);
      // Pass C: t = softmax*g + x, centred; second moment about the exact mean (the
      // two-pass variance of the reference's var_mean lowering).
      float2 q2 = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        if (c.valid(i)) {
          float2 g[H];
          constants(c, 0, i, g);
#pragma unroll
          for (int h = 0; h < H; ++h) {
            const float2 t = fma2(mul2(e[i][h], f2), g[h], x[i][h]);
            e[i][h] = add2(t, nmean);
            q2 = fma2(e[i][h], e[i][h], q2);
          }
        }
      }
      const float var = c.template reduce<SumOp>(q2.x + q2.y) * inv_n;
      const float rstd = rsqrtf(var + p.eps);
      const float2 rstd2 = make_float2(rstd, rstd);
      T* yrow = p.y + r * (long long)c.cols;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        if (c.valid(i)) {
          float2 y[H], ga[H], be[H];
          constants(c, 1, i, ga);
          constants(c, 2, i, be);
#pragma unroll
          for (int h = 0; h < H; ++h) y[h] = fma2(mul2(e[i][h], rstd2), ga[h], be[h]);
          stg_stream(yrow + c.vec_col(i), pack<T>(reinterpret_cast<const float*>(y)));
        }
      }
    }

    // Unaligned rows: per-element validity, scalar fp32, four plain reductions.
    template <class Ctx>
    __device__ __forceinline__ void row_scalar(const Params& p, Ctx& c, long long r,
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
        float2 g[H];
        constants(c, 0, i, g);
        const float* gf = reinterpret_cast<const float*>(g);
#pragma unroll
        for (int j = 0; j < kVec; ++j) {
          x[i][j] = c.ok(i, j) ? fmaf(e[i][j] * inv, gf[j], x[i][j]) : 0.f;
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
        float2 ga[H], be[H];
        float y[kVec];
        constants(c, 1, i, ga);
        constants(c, 2, i, be);
        const float* gaf = reinterpret_cast<const float*>(ga);
        const float* bef = reinterpret_cast<const float*>(be);
#pragma unroll
        for (int j = 0; j < kVec; ++j) y[j] = fmaf(x[i][j] * rstd, gaf[j], bef[j]);
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
  static __host__ __device__ constexpr size_t smem_bytes(int, int) { return 0; }
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
    template <class Ctx>
    __device__ __forceinline__ void init(const Params& p, const Ctx& c, unsigned char*) {
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
  static __host__ __device__ constexpr size_t smem_bytes(int, int) { return 0; }
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
    template <class Ctx>
    __device__ __forceinline__ void init(const Params&, const Ctx&, unsigned char*) {}
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
  static __host__ __device__ constexpr size_t smem_bytes(int, int) { return 0; }
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    T* var;
    T* mean;
    float correction;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }
  template <int VPT> struct Impl {
    template <class Ctx>
    __device__ __forceinline__ void init(const Params&, const Ctx&, unsigned char*) {}
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
  static __host__ __device__ constexpr size_t smem_bytes(int, int) { return 0; }
  static constexpr int kVec = Elem<T>::kVec;
  struct Params {
    const T* x;
    long long* out;
  };
  static __device__ __forceinline__ const T* row_ptr(const Params& p, int) { return p.x; }
  template <int VPT> struct Impl {
    template <class Ctx>
    __device__ __forceinline__ void init(const Params&, const Ctx&, unsigned char*) {}
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
