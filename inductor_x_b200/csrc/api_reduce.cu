// C-ABI entry point of the plain last-axis reductions (persistent row template).
#include "host.h"
#include "ixb/row_bodies.cuh"

namespace {

using ixb_host::aligned16;

template <class Body>
int run(const typename Body::Params& p, int64_t rows, int64_t cols, bool al, const ixb_cfg* user,
        ixb_stream stream) {
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  ixb_cfg cfg = {};
  if (user != nullptr && user->team > 0 && user->vpt > 0) {
    cfg = *user;
    if ((int64_t)cfg.team * cfg.vpt * Body::kVec < cols) return IXB_ERR_SHAPE;
  } else {
    if (!ixb_host::choose_row(cols, sizeof(typename Body::in_t), 8, &cfg)) return IXB_ERR_SHAPE;
    if (user != nullptr) cfg.grid = user->grid;
  }
  if (al) {
    IXB_ROW_DISPATCH(Body, true)
  } else {
    IXB_ROW_DISPATCH(Body, false)
  }
  return IXB_ERR_UNSUPPORTED;
}

template <typename T>
int row_reduce_t(int kind, const void* x, void* out, void* out2, int64_t rows, int64_t cols,
                 float correction, const ixb_cfg* cfg, ixb_stream stream) {
  constexpr int kVec = ixb::Elem<T>::kVec;
  const bool al = cols % kVec == 0 && aligned16(x);
  switch (kind) {
    case IXB_SUM: {
      using B = ixb::RowReduce<T, ixb::kRowSum>;
      return run<B>(typename B::Params{(const T*)x, (T*)out}, rows, cols, al, cfg, stream);
    }
    case IXB_MEAN: {
      using B = ixb::RowReduce<T, ixb::kRowMean>;
      return run<B>(typename B::Params{(const T*)x, (T*)out}, rows, cols, al, cfg, stream);
    }
    case IXB_AMAX: {
      using B = ixb::RowReduce<T, ixb::kRowAmax>;
      return run<B>(typename B::Params{(const T*)x, (T*)out}, rows, cols, al, cfg, stream);
    }
    case IXB_AMIN: {
      using B = ixb::RowReduce<T, ixb::kRowAmin>;
      return run<B>(typename B::Params{(const T*)x, (T*)out}, rows, cols, al, cfg, stream);
    }
    case IXB_ARGMAX: {
      using B = ixb::RowArg<T, true>;
      return run<B>(typename B::Params{(const T*)x, (long long*)out}, rows, cols, al, cfg, stream);
    }
    case IXB_ARGMIN: {
      using B = ixb::RowArg<T, false>;
      return run<B>(typename B::Params{(const T*)x, (long long*)out}, rows, cols, al, cfg, stream);
    }
    case IXB_VAR_MEAN: {
      using B = ixb::RowVarMean<T>;
      if (out2 == nullptr) return IXB_ERR_ARG;
      return run<B>(typename B::Params{(const T*)x, (T*)out, (T*)out2, correction}, rows, cols, al,
                    cfg, stream);
    }
    default:
      return IXB_ERR_ARG;
  }
}

}  // namespace

extern "C" int ixb_row_reduce(int dtype, int kind, const void* x, void* out, void* out2,
                              int64_t rows, int64_t cols, float correction, const ixb_cfg* cfg,
                              ixb_stream stream) {
  if (rows < 0 || cols <= 0) return IXB_ERR_ARG;
  if (rows == 0) return IXB_OK;
  if (x == nullptr || out == nullptr) return IXB_ERR_ARG;
  switch (dtype) {
    case IXB_F32: return row_reduce_t<float>(kind, x, out, out2, rows, cols, correction, cfg, stream);
    case IXB_F16: return row_reduce_t<ixb::f16>(kind, x, out, out2, rows, cols, correction, cfg, stream);
    case IXB_BF16: return row_reduce_t<ixb::bf16>(kind, x, out, out2, rows, cols, correction, cfg, stream);
    default: return IXB_ERR_DTYPE;
  }
}
