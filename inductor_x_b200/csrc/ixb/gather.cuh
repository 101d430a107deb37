// Row gather: out[m, :] = table[idx[m], :]   (index_select / embedding along dim 0).
// The reference leaves this family to extern kernels (inductor_x/lowering.py:89-144,
// 327-339); its generated-code contract for indirect loads is: negative indices wrap and
// an out-of-range index is an error (inductor_x/codegen/triton.py:1666-1710).  The same
// contract holds here, with the error reported through a status word instead of a trap:
// status[0] = 1 and status[1] = the first offending position seen; the row is zero-filled.
//
// Bytes are moved as opaque 128-bit vectors, so the result is bit-exact for any dtype.
// Each thread keeps UNROLL independent row reads in flight; the lanes that share a row
// read the same index word, which the hardware broadcasts.
#pragma once
#include "common.cuh"

namespace ixb {

template <typename IdxT, int UNROLL, bool WRAP_NEGATIVE>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const uint4* __restrict__ table, const IdxT* __restrict__ idx,
                       uint4* __restrict__ out, long long n_rows, long long m, int vec_per_row,
                       int row_shift, long long table_row_vecs, int* __restrict__ status) {
  // row_shift = log2(vec_per_row) when that is a power of two, else -1: splitting a flat
  // vector index into (row, column) must not cost a 64-bit division per vector
  const long long total = m * vec_per_row;
  const bool small = total <= 0x7fffffffLL;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; g < total; g += nthreads * UNROLL) {
    uint4 v[UNROLL];
    long long dst[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const long long gu = g + (long long)u * nthreads;
      dst[u] = -1;
      if (gu < total) {
        long long row;
        if (row_shift >= 0) row = gu >> row_shift;
        else if (small) row = (long long)((unsigned)gu / (unsigned)vec_per_row);
        else row = gu / vec_per_row;
        const int col = (int)(gu - row * vec_per_row);
        long long src = (long long)idx[row];
        if (WRAP_NEGATIVE && src < 0) src += n_rows;
        dst[u] = gu;
        if (src < 0 || src >= n_rows) {
          v[u] = make_uint4(0, 0, 0, 0);
          if (status != nullptr && col == 0 && atomicCAS(status, 0, 1) == 0)
            status[1] = (int)(row < 0x7fffffff ? row : 0x7fffffff);
        } else {
          v[u] = __ldg(table + src * table_row_vecs + col);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u)
      if (dst[u] >= 0) stg_stream(out + dst[u], v[u]);
  }
}

// Fallback for rows that are not a whole number of aligned 128-bit vectors: byte-wise
// elements of ESIZE bytes, one thread per element.
template <typename IdxT, typename E, bool WRAP_NEGATIVE>
__global__ void __launch_bounds__(256)
    gather_rows_elem_kernel(const E* __restrict__ table, const IdxT* __restrict__ idx,
                            E* __restrict__ out, long long n_rows, long long m, long long d,
                            long long table_row_stride, int* __restrict__ status) {
  const long long total = m * d;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= total) return;
  const long long row = g / d, col = g - row * d;
  long long src = (long long)idx[row];
  if (WRAP_NEGATIVE && src < 0) src += n_rows;
  if (src < 0 || src >= n_rows) {
    out[g] = E(0);
    if (status != nullptr && col == 0 && atomicCAS(status, 0, 1) == 0)
      status[1] = (int)(row < 0x7fffffff ? row : 0x7fffffff);
    return;
  }
  out[g] = table[src * table_row_stride + col];
}

}  // namespace ixb
