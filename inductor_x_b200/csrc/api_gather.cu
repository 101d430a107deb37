// C-ABI entry point of the GATHER family.
#include <atomic>
#include "host.h"
#include "ixb/gather.cuh"

namespace {

template <typename IdxT, bool WRAP>
int gather_t(const void* table, const void* idx, void* out, int64_t n_rows, int64_t m,
             int64_t row_bytes, int64_t pitch, int32_t* status, cudaStream_t s) {
  const ixb_devinfo* dev = ixb_host::current_device();
  if (dev == nullptr) return IXB_ERR_CUDA;
  const bool vec_ok = row_bytes % 16 == 0 && pitch % 16 == 0 && ixb_host::aligned16(table) &&
                      ixb_host::aligned16(out);
  if (vec_ok) {
    ixb_problem pb = {};
    pb.family = IXB_FAM_GATHER;
    pb.dtype = IXB_U8;
    pb.outer = m;
    pb.inner = row_bytes;
    ixb_cfg cfg;
    if (int st = ixb_choose_config(&pb, dev, &cfg)) return st;
    const int vpr = (int)(row_bytes / 16);
    int shift = -1;
    if ((vpr & (vpr - 1)) == 0)
      for (shift = 0; (1 << shift) < vpr; ++shift) {}
    // Persistent launch: exactly the CTAs that are resident at once, each striding over the
    // vectors.  A grid of a few waves would leave the last wave partly empty.
    constexpr int kUnroll = 2;
    auto kern = ixb::gather_rows_kernel<IdxT, kUnroll, WRAP>;
    static std::atomic<int> resident[64];   // per device; several host threads may ask at once
    int devid = 0;
    cudaGetDevice(&devid);
    int occ = resident[devid & 63].load(std::memory_order_acquire);
    if (occ == 0) {
      int n = 0;
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, 0) != cudaSuccess || n < 1) n = 1;
      occ = n;
      resident[devid & 63].store(n, std::memory_order_release);
    }
    const long long vecs = (long long)m * vpr;
    long long grid = (vecs + 256LL * kUnroll - 1) / (256LL * kUnroll);
    const long long cap = (long long)dev->sm_count * occ;
    if (grid > cap) grid = cap;
    (void)cfg;
    kern<<<(unsigned)grid, 256, 0, s>>>(
        (const uint4*)table, (const IdxT*)idx, (uint4*)out, n_rows, m, vpr, shift, pitch / 16, status);
    return ixb_host::cuda_status(cudaGetLastError());
  }
  // byte-granular fallback: widest element size dividing the row, pitch and pointers
  const uintptr_t mix = (uintptr_t)table | (uintptr_t)out | (uintptr_t)row_bytes | (uintptr_t)pitch;
  const long long total_b = m * row_bytes;
  auto grid_for = [](long long n) { return (unsigned)((n + 255) / 256); };
  if (mix % 4 == 0) {
    ixb::gather_rows_elem_kernel<IdxT, uint32_t, WRAP><<<grid_for(total_b / 4), 256, 0, s>>>(
        (const uint32_t*)table, (const IdxT*)idx, (uint32_t*)out, n_rows, m, row_bytes / 4,
        pitch / 4, status);
  } else if (mix % 2 == 0) {
    ixb::gather_rows_elem_kernel<IdxT, uint16_t, WRAP><<<grid_for(total_b / 2), 256, 0, s>>>(
        (const uint16_t*)table, (const IdxT*)idx, (uint16_t*)out, n_rows, m, row_bytes / 2,
        pitch / 2, status);
  } else {
    ixb::gather_rows_elem_kernel<IdxT, uint8_t, WRAP><<<grid_for(total_b), 256, 0, s>>>(
        (const uint8_t*)table, (const IdxT*)idx, (uint8_t*)out, n_rows, m, row_bytes, pitch,
        status);
  }
  return ixb_host::cuda_status(cudaGetLastError());
}

}  // namespace

extern "C" int ixb_index_select_rows(const void* table, const void* idx, void* out, int64_t n_rows,
                                     int64_t m, int64_t row_bytes, int64_t table_pitch_bytes,
                                     int idx_dtype, int wrap_negative, int32_t* status,
                                     ixb_stream stream) {
  if (n_rows < 0 || m < 0 || row_bytes < 0 || table_pitch_bytes < row_bytes) return IXB_ERR_ARG;
  if (m == 0 || row_bytes == 0) return IXB_OK;
  if (table == nullptr || idx == nullptr || out == nullptr) return IXB_ERR_ARG;
  if (m * ((row_bytes + 15) / 16) > (1LL << 40)) return IXB_ERR_SHAPE;
  cudaStream_t s = (cudaStream_t)stream;
  if (idx_dtype == IXB_I64) {
    return wrap_negative ? gather_t<long long, true>(table, idx, out, n_rows, m, row_bytes, table_pitch_bytes, status, s)
                         : gather_t<long long, false>(table, idx, out, n_rows, m, row_bytes, table_pitch_bytes, status, s);
  }
  if (idx_dtype == IXB_I32) {
    return wrap_negative ? gather_t<int, true>(table, idx, out, n_rows, m, row_bytes, table_pitch_bytes, status, s)
                         : gather_t<int, false>(table, idx, out, n_rows, m, row_bytes, table_pitch_bytes, status, s);
  }
  return IXB_ERR_DTYPE;
}
