// C-ABI entry points of the context-parallel attention merge kernels.
#include "host.h"
#include "ixb/cp.cuh"

namespace {

// persistent grid: the CTAs that are resident at once, or fewer if the work is smaller
template <class K> long long resident(K kern, const ixb_devinfo* dev) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, 0) != cudaSuccess || n < 1) n = 1;
  return (long long)dev->sm_count * n;
}

template <typename T>
int forward_update_t(const void* prev_attn, const float* prev_max, const float* prev_sum,
                     const void* cur_attn, const float* cur_max, const float* cur_sum, void* out_attn,
                     float* out_max, float* out_sum, int S, int B, int N, int D, int64_t prev_ns,
                     int64_t cur_ns, int64_t out_ns, const ixb_devinfo* dev, cudaStream_t s) {
  auto kern = ixb::cp_forward_update_kernel<T>;
  const size_t smem = (size_t)2 * ixb::kCpRows * N * sizeof(float2);   // weights of two tiles in flight
  if (smem > 48 * 1024) return IXB_ERR_SHAPE;
  const int vph = D / ixb::Elem<T>::kVec;
  int shift = -1;
  if ((vph & (vph - 1)) == 0)
    for (shift = 0; (1 << shift) < vph; ++shift) {}
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, smem) != cudaSuccess || n < 1) n = 1;
  long long grid = (long long)B * ((S + ixb::kCpRows - 1) / ixb::kCpRows);
  const long long cap = (long long)dev->sm_count * n;
  if (grid > cap) grid = cap;
  kern<<<(unsigned)grid, 256, smem, s>>>((const T*)prev_attn, prev_max, prev_sum, (const T*)cur_attn, cur_max,
                                        cur_sum, (T*)out_attn, out_max, out_sum, S, B, N, D, prev_ns, cur_ns,
                                        out_ns, shift);
  return ixb_host::cuda_status(cudaGetLastError());
}

template <typename T>
int accumulate_t(void* acc, const void* cur, int64_t numel, const ixb_devinfo* dev, cudaStream_t s) {
  constexpr int kVec = ixb::Elem<T>::kVec;
  if (numel % kVec != 0) return IXB_ERR_ALIGN;
  auto kern = ixb::accumulate_kernel<T>;
  const long long nvec = numel / kVec;
  long long grid = (nvec + 255) / 256;
  const long long cap = resident(kern, dev);
  if (grid > cap) grid = cap;
  kern<<<(unsigned)grid, 256, 0, s>>>((T*)acc, (const T*)cur, nvec);
  return ixb_host::cuda_status(cudaGetLastError());
}

}  // namespace

extern "C" int ixb_cp_forward_update(int dtype, const void* prev_attn, const float* prev_max,
                                     const float* prev_sum, const void* cur_attn, const float* cur_max,
                                     const float* cur_sum, void* out_attn, float* out_max, float* out_sum,
                                     int32_t S, int32_t B, int32_t N, int32_t D,
                                     int64_t prev_stat_nstride, int64_t cur_stat_nstride,
                                     int64_t out_stat_nstride, ixb_stream stream) {
  if (!prev_attn || !prev_max || !prev_sum || !cur_attn || !cur_max || !cur_sum || !out_attn || !out_max ||
      !out_sum || S < 0 || B < 0 || N <= 0 || D <= 0)
    return IXB_ERR_ARG;
  if (S == 0 || B == 0) return IXB_OK;
  const int es = ixb_host::elem_size(dtype);
  if (dtype != IXB_F32 && dtype != IXB_F16 && dtype != IXB_BF16) return IXB_ERR_DTYPE;
  if (((int64_t)D * es) % 16 != 0 || !ixb_host::aligned16(prev_attn) || !ixb_host::aligned16(cur_attn) ||
      !ixb_host::aligned16(out_attn) || !ixb_host::aligned16(prev_max) || !ixb_host::aligned16(prev_sum) ||
      !ixb_host::aligned16(cur_max) || !ixb_host::aligned16(cur_sum) || !ixb_host::aligned16(out_max) ||
      !ixb_host::aligned16(out_sum) || prev_stat_nstride % 4 || cur_stat_nstride % 4 || out_stat_nstride % 4)
    return IXB_ERR_ALIGN;
  if ((int64_t)N * D > 0x7fffffffLL) return IXB_ERR_SHAPE;
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case IXB_BF16:
      return forward_update_t<ixb::bf16>(prev_attn, prev_max, prev_sum, cur_attn, cur_max, cur_sum, out_attn,
                                         out_max, out_sum, S, B, N, D, prev_stat_nstride, cur_stat_nstride,
                                         out_stat_nstride, dev, s);
    case IXB_F16:
      return forward_update_t<ixb::f16>(prev_attn, prev_max, prev_sum, cur_attn, cur_max, cur_sum, out_attn,
                                        out_max, out_sum, S, B, N, D, prev_stat_nstride, cur_stat_nstride,
                                        out_stat_nstride, dev, s);
    default:
      return forward_update_t<float>(prev_attn, prev_max, prev_sum, cur_attn, cur_max, cur_sum, out_attn,
                                     out_max, out_sum, S, B, N, D, prev_stat_nstride, cur_stat_nstride,
                                     out_stat_nstride, dev, s);
  }
}

extern "C" int ixb_cp_forward_update_lse(float* prev_attn, float* prev_lse, const float* cur_attn,
                                         const float* cur_lse, int32_t B, int32_t N, int32_t S, int32_t D,
                                         int64_t prev_attn_nstride, int64_t prev_lse_nstride,
                                         int64_t cur_attn_nstride, int64_t cur_lse_nstride,
                                         ixb_stream stream) {
  if (!prev_attn || !prev_lse || !cur_attn || !cur_lse || B < 0 || N < 0 || S < 0 || D <= 0) return IXB_ERR_ARG;
  if (B == 0 || N == 0 || S == 0) return IXB_OK;
  if (D % 4 != 0 || !ixb_host::aligned16(prev_attn) || !ixb_host::aligned16(cur_attn) ||
      prev_attn_nstride % 4 || cur_attn_nstride % 4)
    return IXB_ERR_ALIGN;
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  auto kern = ixb::cp_forward_update_lse_kernel;
  const long long rows = (long long)B * N * S;
  long long grid = (rows + 7) / 8;  // eight warps, one row each, per CTA
  const long long cap = resident(kern, dev);
  if (grid > cap) grid = cap;
  kern<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(prev_attn, prev_lse, cur_attn, cur_lse, B * N, S, D,
                                                        prev_attn_nstride, prev_lse_nstride,
                                                        cur_attn_nstride, cur_lse_nstride);
  return ixb_host::cuda_status(cudaGetLastError());
}

extern "C" int ixb_cp_accumulate(int dtype, void* acc, const void* cur, int64_t numel, ixb_stream stream) {
  if (!acc || !cur || numel < 0) return IXB_ERR_ARG;
  if (numel == 0) return IXB_OK;
  if (!ixb_host::aligned16(acc) || !ixb_host::aligned16(cur)) return IXB_ERR_ALIGN;
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case IXB_BF16: return accumulate_t<ixb::bf16>(acc, cur, numel, dev, s);
    case IXB_F16: return accumulate_t<ixb::f16>(acc, cur, numel, dev, s);
    case IXB_F32: return accumulate_t<float>(acc, cur, numel, dev, s);
    default: return IXB_ERR_DTYPE;
  }
}
