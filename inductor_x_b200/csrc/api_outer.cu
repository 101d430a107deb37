// C-ABI entry points of the OUTER and SHORT_ROW reduction families.
#include "host.h"
#include "ixb/outer.cuh"
#include "ixb/short_row.cuh"

namespace {

using ixb_host::aligned16;

template <typename T, typename OutT, class Op, int VC>
cudaError_t launch_outer_vc(const T* x, OutT* dst, int64_t outer, int64_t R, int64_t inner,
                            int chunks, int rsplit, int64_t seg_stride, float post,
                            cudaStream_t s) {
  const long long grid = outer * chunks * rsplit;
  ixb::outer_reduce_kernel<T, OutT, Op, 256, VC, 8>
      <<<(unsigned)grid, 256, 0, s>>>(x, dst, R, inner, chunks, rsplit, seg_stride, post);
  return cudaGetLastError();
}

template <typename T, typename OutT, class Op>
cudaError_t launch_outer(const T* x, OutT* dst, int64_t outer, int64_t R, int64_t inner, int vc,
                         int chunks, int rsplit, int64_t seg_stride, float post, cudaStream_t s) {
  switch (vc) {
    case 1: return launch_outer_vc<T, OutT, Op, 1>(x, dst, outer, R, inner, chunks, rsplit, seg_stride, post, s);
    case 2: return launch_outer_vc<T, OutT, Op, 2>(x, dst, outer, R, inner, chunks, rsplit, seg_stride, post, s);
    case 4: return launch_outer_vc<T, OutT, Op, 4>(x, dst, outer, R, inner, chunks, rsplit, seg_stride, post, s);
    case 8: return launch_outer_vc<T, OutT, Op, 8>(x, dst, outer, R, inner, chunks, rsplit, seg_stride, post, s);
    case 16: return launch_outer_vc<T, OutT, Op, 16>(x, dst, outer, R, inner, chunks, rsplit, seg_stride, post, s);
    default: return launch_outer_vc<T, OutT, Op, 32>(x, dst, outer, R, inner, chunks, rsplit, seg_stride, post, s);
  }
}

template <typename T, class Op>
int outer_reduce_op(const void* x, void* out, int64_t outer, int64_t R, int64_t inner,
                    void* scratch, size_t scratch_bytes, const ixb_cfg* user, float post,
                    ixb_stream stream) {
  constexpr int kVec = ixb::Elem<T>::kVec;
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t out_numel = outer * inner;
  if (out_numel == 0) return IXB_OK;
  if (inner % kVec != 0 || !aligned16(x)) {
    const long long grid = (out_numel + 255) / 256;
    ixb::outer_reduce_scalar_kernel<T, Op>
        <<<(unsigned)grid, 256, 0, s>>>((const T*)x, (T*)out, R, inner, out_numel, post);
    return ixb_host::cuda_status(cudaGetLastError());
  }
  ixb_cfg cfg = {};
  ixb_problem pb = {};
  pb.family = IXB_FAM_OUTER;
  pb.dtype = sizeof(T) == 4 ? IXB_F32 : IXB_F16;
  pb.outer = outer;
  pb.reduce = R;
  pb.inner = inner;
  if (int st = ixb_choose_config(&pb, ixb_host::current_device(), &cfg)) return st;
  if (user != nullptr && user->rsplit > 0) cfg.rsplit = user->rsplit;
  const int vc = cfg.vpt;
  const int64_t nv = inner / kVec;
  const int chunks = (int)((nv + vc - 1) / vc);
  int rsplit = cfg.rsplit;
  if (rsplit > R) rsplit = (int)R;
  if (rsplit < 1) rsplit = 1;
  if (outer * chunks * rsplit > 0x7fffffffLL) return IXB_ERR_SHAPE;
  if (rsplit == 1) {
    return ixb_host::cuda_status(launch_outer<T, T, Op>((const T*)x, (T*)out, outer, R, inner, vc,
                                                         chunks, 1, 0, post, s));
  }
  const size_t need = ixb_outer_reduce_scratch_bytes(outer, inner, rsplit);
  if (scratch == nullptr || scratch_bytes < need) return IXB_ERR_SCRATCH;
  cudaError_t e = launch_outer<T, float, Op>((const T*)x, (float*)scratch, outer, R, inner, vc,
                                             chunks, rsplit, out_numel, 1.f, s);
  if (e != cudaSuccess) return ixb_host::cuda_status(e);
  const long long grid = (out_numel + 255) / 256;
  ixb::outer_reduce_finalize_kernel<T, Op>
      <<<(unsigned)grid, 256, 0, s>>>((const float*)scratch, (T*)out, out_numel, rsplit, post);
  return ixb_host::cuda_status(cudaGetLastError());
}

template <typename T>
int outer_reduce_t(int kind, const void* x, void* out, int64_t outer, int64_t R, int64_t inner,
                   void* scratch, size_t scratch_bytes, const ixb_cfg* cfg, ixb_stream stream) {
  switch (kind) {
    case IXB_SUM:
      return outer_reduce_op<T, ixb::SumOp>(x, out, outer, R, inner, scratch, scratch_bytes, cfg, 1.f, stream);
    case IXB_MEAN:
      return outer_reduce_op<T, ixb::SumOp>(x, out, outer, R, inner, scratch, scratch_bytes, cfg, 1.f / (float)R, stream);
    case IXB_AMAX:
      return outer_reduce_op<T, ixb::MaxOp>(x, out, outer, R, inner, scratch, scratch_bytes, cfg, 1.f, stream);
    case IXB_AMIN:
      return outer_reduce_op<T, ixb::MinOp>(x, out, outer, R, inner, scratch, scratch_bytes, cfg, 1.f, stream);
    default:
      return IXB_ERR_UNSUPPORTED;
  }
}

template <typename T, class Op, int LG>
int short_row_lg(const void* x, void* out, int64_t A, int64_t B, int64_t C, int64_t sa, int64_t sb,
                 int64_t sc, float post, cudaStream_t s) {
  constexpr int TB = 32, TC = 32;
  const int64_t tiles_b = (B + TB - 1) / TB, tiles_c = (C + TC - 1) / TC;
  const int64_t grid = A * tiles_b * tiles_c;
  if (grid == 0) return IXB_OK;
  if (grid > 0x7fffffffLL) return IXB_ERR_SHAPE;
  ixb::short_row_reduce_kernel<T, Op, LG, TB, TC, 256><<<(unsigned)grid, 256, 0, s>>>(
      (const T*)x, (T*)out, (int)B, (int)C, sa, sb, sc, (int)tiles_b, (int)tiles_c, post);
  return ixb_host::cuda_status(cudaGetLastError());
}

template <typename T, class Op>
int short_row_op(const void* x, void* out, int64_t A, int64_t B, int64_t C, int64_t L, int64_t sa,
                 int64_t sb, int64_t sc, float post, ixb_stream stream) {
  constexpr int kVec = ixb::Elem<T>::kVec;
  cudaStream_t s = (cudaStream_t)stream;
  if (L % kVec != 0 || !aligned16(x)) return IXB_ERR_ALIGN;
  switch (L / kVec) {
    case 1: return short_row_lg<T, Op, 1>(x, out, A, B, C, sa, sb, sc, post, s);
    case 2: return short_row_lg<T, Op, 2>(x, out, A, B, C, sa, sb, sc, post, s);
    case 4: return short_row_lg<T, Op, 4>(x, out, A, B, C, sa, sb, sc, post, s);
    case 8: return short_row_lg<T, Op, 8>(x, out, A, B, C, sa, sb, sc, post, s);
    case 16: return short_row_lg<T, Op, 16>(x, out, A, B, C, sa, sb, sc, post, s);
    case 32: return short_row_lg<T, Op, 32>(x, out, A, B, C, sa, sb, sc, post, s);
    default: return IXB_ERR_SHAPE;
  }
}

template <typename T>
int short_row_t(int kind, const void* x, void* out, int64_t A, int64_t B, int64_t C, int64_t L,
                int64_t sa, int64_t sb, int64_t sc, ixb_stream stream) {
  switch (kind) {
    case IXB_SUM: return short_row_op<T, ixb::SumOp>(x, out, A, B, C, L, sa, sb, sc, 1.f, stream);
    case IXB_MEAN: return short_row_op<T, ixb::SumOp>(x, out, A, B, C, L, sa, sb, sc, 1.f / (float)L, stream);
    case IXB_AMAX: return short_row_op<T, ixb::MaxOp>(x, out, A, B, C, L, sa, sb, sc, 1.f, stream);
    case IXB_AMIN: return short_row_op<T, ixb::MinOp>(x, out, A, B, C, L, sa, sb, sc, 1.f, stream);
    default: return IXB_ERR_UNSUPPORTED;
  }
}

}  // namespace

extern "C" {

size_t ixb_outer_reduce_scratch_bytes(int64_t outer, int64_t inner, int rsplit) {
  if (rsplit <= 1 || outer <= 0 || inner <= 0) return 0;
  // extents whose product does not fit are answered with the largest size: no buffer satisfies it
  const size_t cap = SIZE_MAX / sizeof(float);
  if ((size_t)inner > cap / (size_t)outer || (size_t)rsplit > cap / ((size_t)outer * (size_t)inner)) return SIZE_MAX;
  return (size_t)outer * (size_t)inner * (size_t)rsplit * sizeof(float);
}

int ixb_outer_reduce(int dtype, int kind, const void* x, void* out, int64_t outer, int64_t R,
                     int64_t inner, void* scratch, size_t scratch_bytes, const ixb_cfg* cfg,
                     ixb_stream stream) {
  if (outer < 0 || R <= 0 || inner < 0) return IXB_ERR_ARG;
  if (outer == 0 || inner == 0) return IXB_OK;
  if (x == nullptr || out == nullptr) return IXB_ERR_ARG;
  // outer * inner outputs, one thread each in the scalar paths: must fit a 32-bit grid of 256-thread CTAs
  if (inner > (0x7fffffffLL * 256) / outer) return IXB_ERR_SHAPE;
  switch (dtype) {
    case IXB_F32: return outer_reduce_t<float>(kind, x, out, outer, R, inner, scratch, scratch_bytes, cfg, stream);
    case IXB_F16: return outer_reduce_t<ixb::f16>(kind, x, out, outer, R, inner, scratch, scratch_bytes, cfg, stream);
    case IXB_BF16: return outer_reduce_t<ixb::bf16>(kind, x, out, outer, R, inner, scratch, scratch_bytes, cfg, stream);
    default: return IXB_ERR_DTYPE;
  }
}

int ixb_short_row_reduce(int dtype, int kind, const void* x, void* out, int64_t A, int64_t B,
                         int64_t C, int64_t L, int64_t sa, int64_t sb, int64_t sc,
                         ixb_stream stream) {
  if (A < 0 || B < 0 || C < 0 || L <= 0) return IXB_ERR_ARG;
  if (A == 0 || B == 0 || C == 0) return IXB_OK;
  if (x == nullptr || out == nullptr) return IXB_ERR_ARG;
  switch (dtype) {
    case IXB_F32: return short_row_t<float>(kind, x, out, A, B, C, L, sa, sb, sc, stream);
    case IXB_F16: return short_row_t<ixb::f16>(kind, x, out, A, B, C, L, sa, sb, sc, stream);
    case IXB_BF16: return short_row_t<ixb::bf16>(kind, x, out, A, B, C, L, sa, sb, sc, stream);
    default: return IXB_ERR_DTYPE;
  }
}

}  // extern "C"
