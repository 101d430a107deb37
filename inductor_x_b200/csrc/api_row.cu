// C-ABI entry points of the fused ROW-family graphs (persistent row template).
#include "host.h"
#include "ixb/row_bodies.cuh"

namespace {

using ixb_host::aligned16;

// Resolve the launch configuration: the caller's, or the chooser's.
int resolve_cfg(const ixb_cfg* user, int64_t cols, int elsize, int max_vpt, ixb_cfg* cfg) {
  if (user != nullptr && user->team > 0 && user->vpt > 0) {
    *cfg = *user;
    const int64_t vec = 16 / elsize;
    if ((int64_t)cfg->team * cfg->vpt * vec < cols) return IXB_ERR_SHAPE;
    return IXB_OK;
  }
  ixb_cfg c = {};
  if (!ixb_host::choose_row(cols, elsize, max_vpt, &c)) return IXB_ERR_SHAPE;
  if (user != nullptr) c.grid = user->grid;
  *cfg = c;
  return IXB_OK;
}

template <typename T>
int softmax_layernorm_t(const void* x, const void* g, const void* gamma, const void* beta, void* y,
                        int64_t rows, int64_t cols, float eps, const ixb_cfg* user,
                        ixb_stream stream) {
  using Body = ixb::SoftmaxLayerNorm<T>;
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  ixb_cfg cfg;
  if (int st = resolve_cfg(user, cols, sizeof(T), 4, &cfg)) return st;
  typename Body::Params p{(const T*)x, (const T*)g, (const T*)gamma, (const T*)beta, (T*)y, eps};
  const bool al = cols % Body::kVec == 0 && aligned16(x) && aligned16(g) && aligned16(gamma) &&
                  aligned16(beta) && aligned16(y);
  if (al) {
    IXB_ROW_DISPATCH(Body, true)
  } else {
    IXB_ROW_DISPATCH(Body, false)
  }
  return IXB_ERR_UNSUPPORTED;
}

template <typename T, bool RES>
int rmsnorm_t(const void* x, const void* res, const void* w, void* y, void* h_out, int64_t rows,
              int64_t cols, float eps, const ixb_cfg* user, ixb_stream stream) {
  using Body = ixb::RmsNorm<T, RES>;
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  ixb_cfg cfg;
  if (int st = resolve_cfg(user, cols, sizeof(T), 4, &cfg)) return st;
  typename Body::Params p{(const T*)x, (const T*)res, (const T*)w, (T*)y, (T*)h_out, eps};
  const bool al = cols % Body::kVec == 0 && aligned16(x) && aligned16(res) && aligned16(w) &&
                  aligned16(y) && aligned16(h_out);
  if (al) {
    IXB_ROW_DISPATCH(Body, true)
  } else {
    IXB_ROW_DISPATCH(Body, false)
  }
  return IXB_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" {

int ixb_affine_gelu_rowsum_f32(const float* x, const float* w, const float* b, float* out,
                               int64_t rows, int64_t cols, const ixb_cfg* user,
                               ixb_stream stream) {
  using Body = ixb::AffineGeluRowSum;
  if (rows < 0 || cols <= 0) return IXB_ERR_ARG;
  if (rows == 0) return IXB_OK;
  if (x == nullptr || w == nullptr || b == nullptr || out == nullptr) return IXB_ERR_ARG;
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  ixb_cfg cfg;
  // two vectors per thread keep w and b in registers (measured 9.1 us vs 11.6 us at four
  // vectors per thread on 8192 x 1024); longer rows fall back to the general choice
  if (resolve_cfg(user, cols, 4, 2, &cfg) != IXB_OK) {
    if (int st = resolve_cfg(user, cols, 4, 8, &cfg)) return st;
  }
  Body::Params p{x, w, b, out};
  const bool al = cols % 4 == 0 && aligned16(x) && aligned16(w) && aligned16(b);
  if (al) {
    IXB_ROW_DISPATCH(Body, true)
  } else {
    IXB_ROW_DISPATCH(Body, false)
  }
  return IXB_ERR_UNSUPPORTED;
}

int ixb_softmax_layernorm(int dtype, const void* x, const void* g, const void* gamma,
                          const void* beta, void* y, int64_t rows, int64_t cols, float eps,
                          const ixb_cfg* cfg, ixb_stream stream) {
  if (rows < 0 || cols <= 0) return IXB_ERR_ARG;
  if (rows == 0) return IXB_OK;
  if (!x || !g || !gamma || !beta || !y) return IXB_ERR_ARG;
  switch (dtype) {
    case IXB_BF16:
      return softmax_layernorm_t<ixb::bf16>(x, g, gamma, beta, y, rows, cols, eps, cfg, stream);
    case IXB_F16:
      return softmax_layernorm_t<ixb::f16>(x, g, gamma, beta, y, rows, cols, eps, cfg, stream);
    case IXB_F32:
      return softmax_layernorm_t<float>(x, g, gamma, beta, y, rows, cols, eps, cfg, stream);
    default:
      return IXB_ERR_DTYPE;
  }
}

int ixb_rmsnorm(int dtype, const void* x, const void* res, const void* w, void* y, void* h_out,
                int64_t rows, int64_t cols, float eps, const ixb_cfg* cfg, ixb_stream stream) {
  if (rows < 0 || cols <= 0) return IXB_ERR_ARG;
  if (rows == 0) return IXB_OK;
  if (!x || !w || !y) return IXB_ERR_ARG;
  if (res == nullptr && h_out != nullptr) return IXB_ERR_ARG;
  switch (dtype) {
    case IXB_BF16:
      return res ? rmsnorm_t<ixb::bf16, true>(x, res, w, y, h_out, rows, cols, eps, cfg, stream)
                 : rmsnorm_t<ixb::bf16, false>(x, res, w, y, h_out, rows, cols, eps, cfg, stream);
    case IXB_F16:
      return res ? rmsnorm_t<ixb::f16, true>(x, res, w, y, h_out, rows, cols, eps, cfg, stream)
                 : rmsnorm_t<ixb::f16, false>(x, res, w, y, h_out, rows, cols, eps, cfg, stream);
    case IXB_F32:
      return res ? rmsnorm_t<float, true>(x, res, w, y, h_out, rows, cols, eps, cfg, stream)
                 : rmsnorm_t<float, false>(x, res, w, y, h_out, rows, cols, eps, cfg, stream);
    default:
      return IXB_ERR_DTYPE;
  }
}

}  // extern "C"
