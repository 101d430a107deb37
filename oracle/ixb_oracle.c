/*
 * Plain-C restatement of the hot-path math with double accumulation.
 * TEST INFRASTRUCTURE ONLY: built by oracle/Makefile into oracle/_build/ and loaded by
 * tests, smoke() and the CPU-baseline legs of bench.py.  The product never links it.
 *
 * The reference has no CPU code of its own for these graphs (its arithmetic is generated
 * Ascend Triton); each function restates the graph the reference's lowerings define, with
 * the file:line it follows, independently of torch's kernels so that the two oracles can
 * be checked against each other.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <string.h>

/* out[r] = sum_c gelu_erf(x*w+b): mul lowering inductor_x/lowering.py:251-268, sum with
 * wide accumulation inductor_x/lowering.py:204-215; erf GELU = torch's default. */
void orc_affine_gelu_rowsum(const float* x, const float* w, const float* b, double* out,
                            int64_t rows, int64_t cols) {
  for (int64_t r = 0; r < rows; ++r) {
    double acc = 0.0;
    for (int64_t c = 0; c < cols; ++c) {
      /* the product and sum are fp32 in the graph (inputs are fp32 tensors) */
      const float v = x[r * cols + c] * w[c] + b[c];
      acc += 0.5 * (double)v * (1.0 + erf((double)v * 0.70710678118654752440));
    }
    out[r] = acc;
  }
}

/* y = layer_norm(softmax(x)*g + x): softmax as max / exp / sum; mean then centred second
 * moment (two-pass variance of inductor_x/lowering.py:270-325); inputs already widened
 * to fp32 (inductor_x/codegen/triton.py:1431-1433). */
void orc_softmax_layernorm(const float* x, const float* g, const float* gamma, const float* beta,
                           double* y, int64_t rows, int64_t cols, double eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* xr = x + r * cols;
    double* yr = y + r * cols;
    double m = -INFINITY, s = 0.0, mean = 0.0, var = 0.0;
    for (int64_t c = 0; c < cols; ++c) if (xr[c] > m) m = xr[c];
    for (int64_t c = 0; c < cols; ++c) { yr[c] = exp((double)xr[c] - m); s += yr[c]; }
    for (int64_t c = 0; c < cols; ++c) { yr[c] = yr[c] / s * g[c] + xr[c]; mean += yr[c]; }
    mean /= (double)cols;
    for (int64_t c = 0; c < cols; ++c) { const double d = yr[c] - mean; var += d * d; }
    var /= (double)cols;
    const double rstd = 1.0 / sqrt(var + eps);
    for (int64_t c = 0; c < cols; ++c) yr[c] = (yr[c] - mean) * rstd * gamma[c] + beta[c];
  }
}

/* kind: 0 sum, 1 mean, 2 amax, 3 amin.  x is [outer, R, inner]; R is reduced
 * (high-order reduction, inductor_x/codegen/triton.py:1003-1031). */
void orc_reduce_mid(const float* x, double* out, int64_t outer, int64_t R, int64_t inner, int kind) {
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      double a = kind == 2 ? -INFINITY : (kind == 3 ? INFINITY : 0.0);
      for (int64_t r = 0; r < R; ++r) {
        const double v = x[(o * R + r) * inner + i];
        if (kind == 2) { if (v > a || v != v) a = v; }
        else if (kind == 3) { if (v < a || v != v) a = v; }
        else a += v;
        if (a != a) break; /* NaN propagates */
      }
      if (kind == 1) a /= (double)R;
      out[o * inner + i] = a;
    }
}

/* Bit-exact row gather with the contract of the reference's indirect loads
 * (inductor_x/codegen/triton.py:1666-1710): optional negative wrap; an out-of-range index
 * returns its position + 1 and zero-fills the row. */
int64_t orc_index_select_rows(const uint8_t* table, const int64_t* idx, uint8_t* out,
                              int64_t n_rows, int64_t m, int64_t row_bytes, int wrap_negative) {
  int64_t bad = 0;
  for (int64_t i = 0; i < m; ++i) {
    int64_t s = idx[i];
    if (wrap_negative && s < 0) s += n_rows;
    if (s < 0 || s >= n_rows) {
      memset(out + i * row_bytes, 0, (size_t)row_bytes);
      if (!bad) bad = i + 1;
      continue;
    }
    memcpy(out + i * row_bytes, table + s * row_bytes, (size_t)row_bytes);
  }
  return bad;
}

/* softmax(q k^T * scale [causal]) v for one [S, D] head, double arithmetic; the graph of
 * inductor_x/npu_fusion_attention_graph.py:140-147 with scale = 1/inv_scale_factor.
 * lse[i] = log sum_j exp(s_ij). */
void orc_attention_head(const float* q, const float* k, const float* v, double* out, double* lse,
                        int64_t Sq, int64_t Sk, int64_t D, double scale, int causal) {
  for (int64_t i = 0; i < Sq; ++i) {
    const int64_t jmax = causal ? (i + (Sk - Sq) + 1) : Sk;
    double m = -INFINITY;
    for (int64_t j = 0; j < jmax && j < Sk; ++j) {
      double s = 0.0;
      for (int64_t d = 0; d < D; ++d) s += (double)q[i * D + d] * (double)k[j * D + d];
      s *= scale;
      if (s > m) m = s;
    }
    double denom = 0.0;
    for (int64_t d = 0; d < D; ++d) out[i * D + d] = 0.0;
    for (int64_t j = 0; j < jmax && j < Sk; ++j) {
      double s = 0.0;
      for (int64_t d = 0; d < D; ++d) s += (double)q[i * D + d] * (double)k[j * D + d];
      const double p = exp(s * scale - m);
      denom += p;
      for (int64_t d = 0; d < D; ++d) out[i * D + d] += p * (double)v[j * D + d];
    }
    for (int64_t d = 0; d < D; ++d) out[i * D + d] /= denom;
    lse[i] = m + log(denom);
  }
}
