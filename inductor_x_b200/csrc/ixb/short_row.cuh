// Short-row reduction with a permuted store.  x is contiguous [A][B][C][L] with a short
// stride-1 axis L (at most 32 vectors of 128 bits) that is reduced; the result is stored
// at out[a*sa + b*sb + c*sc].  When sb == 1 the output is the transpose of the read order
// within each `a` slab - the case the reference handles with a second set of index
// variables and a tile permute (inductor_x/codegen/triton.py:856-888,1303-1332).  Here a
// CTA reduces a TB x TC tile of rows, parks the TB*TC results in shared memory and writes
// them back along the output's stride-1 axis, so both sides move whole sectors.
//
// LG lanes (L / vector width, a power of two) cooperate on one row; a warp-wide load
// covers 32/LG consecutive rows = 512 contiguous bytes.
#pragma once
#include "common.cuh"

namespace ixb {

template <typename T, class Op, int LG, int TB, int TC, int THREADS>
__global__ void __launch_bounds__(THREADS)
    short_row_reduce_kernel(const T* __restrict__ x, T* __restrict__ out, int B, int C,
                            long long sa, long long sb, long long sc, int tiles_b, int tiles_c,
                            float post_scale) {
  constexpr int kVec = Elem<T>::kVec;
  constexpr int L = LG * kVec;
  constexpr int ROWS_PER_WARP = 32 / LG;
  constexpr int WARPS = THREADS / 32;
  static_assert(TC % ROWS_PER_WARP == 0, "tile width must be a multiple of rows per warp load");
  constexpr int STEPS_C = TC / ROWS_PER_WARP;
  __shared__ float tile[TB][TC + 1];

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / LG;       // which of the warp's rows
  const int lv = lane % LG;        // vector inside the row

  int t = blockIdx.x;
  const int tc = t % tiles_c;
  t /= tiles_c;
  const int tb = t % tiles_b;
  const long long a = t / tiles_b;
  const int b0 = tb * TB, c0 = tc * TC;

  // (bl, step) pairs of the tile are dealt round-robin to the warps
  constexpr int ITEMS = TB * STEPS_C;
  constexpr int UNROLL = 4;
  for (int it0 = warp; it0 < ITEMS; it0 += WARPS * UNROLL) {
    uint4 raw[UNROLL];
    bool ok[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int it = it0 + u * WARPS;
      const int bl = it / STEPS_C, cl = (it % STEPS_C) * ROWS_PER_WARP + sub;
      ok[u] = it < ITEMS && (b0 + bl) < B && (c0 + cl) < C;
      if (ok[u]) {
        const long long row = (a * B + (b0 + bl)) * C + (c0 + cl);
        raw[u] = ldg_stream(x + row * L + lv * kVec);
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int it = it0 + u * WARPS;
      float acc = Op::identity();
      if (ok[u]) {
        float f[kVec];
        unpack<T>(raw[u], f);
#pragma unroll
        for (int j = 0; j < kVec; ++j) acc = Op::combine(acc, f[j]);
      }
      acc = lane_group_reduce<Op, LG>(acc);
      if (it < ITEMS && lv == 0) {
        const int bl = it / STEPS_C, cl = (it % STEPS_C) * ROWS_PER_WARP + sub;
        tile[bl][cl] = acc * post_scale;
      }
    }
  }
  __syncthreads();
  // write-back along the output's stride-1 axis
  if (sb == 1) {
    for (int e = threadIdx.x; e < TB * TC; e += THREADS) {
      const int bl = e % TB, cl = e / TB;
      if (b0 + bl < B && c0 + cl < C)
        out[a * sa + (long long)(b0 + bl) * sb + (long long)(c0 + cl) * sc] =
            Elem<T>::from_f(tile[bl][cl]);
    }
  } else {
    for (int e = threadIdx.x; e < TB * TC; e += THREADS) {
      const int cl = e % TC, bl = e / TC;
      if (b0 + bl < B && c0 + cl < C)
        out[a * sa + (long long)(b0 + bl) * sb + (long long)(c0 + cl) * sc] =
            Elem<T>::from_f(tile[bl][cl]);
    }
  }
}

}  // namespace ixb
