// Outer ("high-order") reduction template: x is contiguous [outer][R][inner] and the
// middle axis R is reduced, so the output [outer][inner] keeps the stride-1 axis.  This
// is the family the reference emits as a [RBLOCK, XBLOCK_SUB] tile reduced along dim 0
// (inductor_x/codegen/triton.py:1003-1031) and, for very long R, splits with atomics
// (inductor_x/codegen/split_tiling.py:159-165).  Here the split is deterministic:
// partial results go to caller-provided scratch and a second launch folds them.
//
// A CTA owns VC consecutive 128-bit vectors of the inner axis for one outer index and one
// R segment.  Threads form a (TY x VC) grid; a warp therefore reads 32/VC consecutive
// rows x VC vectors, which is one contiguous 512-byte span whenever VC covers the inner
// axis.  Each thread keeps UNROLL independent loads in flight.
#pragma once
#include "common.cuh"

namespace ixb {

// OutT is T for a single-stage launch and float when partials go to scratch
// (dst = scratch, seg_stride = number of output elements).
template <typename T, typename OutT, class Op, int THREADS, int VC, int UNROLL>
__global__ void __launch_bounds__(THREADS)
    outer_reduce_kernel(const T* __restrict__ x, OutT* __restrict__ dst, long long R,
                        long long inner, int chunks, int rsplit, long long seg_stride,
                        float post_scale) {
  constexpr int kVec = Elem<T>::kVec;
  constexpr int TY = THREADS / VC;
  __shared__ float part[TY][VC * kVec + 1];

  const int tx = threadIdx.x % VC;
  const int ty = threadIdx.x / VC;
  // blockIdx.x = ((outer * chunks) + chunk) * rsplit + seg
  const int seg = blockIdx.x % rsplit;
  const long long oc = blockIdx.x / rsplit;
  const int chunk = (int)(oc % chunks);
  const long long o = oc / chunks;

  const long long nv = inner / kVec;
  const long long v = (long long)chunk * VC + tx;
  const bool live = v < nv;

  const long long seg_len = (R + rsplit - 1) / rsplit;
  const long long r0 = seg * seg_len;
  const long long r1 = (r0 + seg_len < R) ? r0 + seg_len : R;

  float acc[kVec];
#pragma unroll
  for (int j = 0; j < kVec; ++j) acc[j] = Op::identity();

  if (live) {
    const T* base = x + (o * R) * inner + v * kVec;
    long long r = r0 + ty;
    for (; r + (long long)(UNROLL - 1) * TY < r1; r += (long long)UNROLL * TY) {
      uint4 raw[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) raw[u] = ldg_stream(base + (r + (long long)u * TY) * inner);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        float f[kVec];
        unpack<T>(raw[u], f);
#pragma unroll
        for (int j = 0; j < kVec; ++j) acc[j] = Op::combine(acc[j], f[j]);
      }
    }
    for (; r < r1; r += TY) {
      float f[kVec];
      unpack<T>(ldg_stream(base + r * inner), f);
#pragma unroll
      for (int j = 0; j < kVec; ++j) acc[j] = Op::combine(acc[j], f[j]);
    }
  }
#pragma unroll
  for (int j = 0; j < kVec; ++j) part[ty][tx * kVec + j] = acc[j];
  __syncthreads();

  // fold the TY partial rows: one thread per output element of the chunk
  for (int e = threadIdx.x; e < VC * kVec; e += THREADS) {
    const long long col = (long long)chunk * VC * kVec + e;
    if (col >= inner) continue;
    float a = part[0][e];
#pragma unroll 4
    for (int y = 1; y < TY; ++y) a = Op::combine(a, part[y][e]);
    dst[(long long)seg * seg_stride + o * inner + col] = Elem<OutT>::from_f(a * post_scale);
  }
}

// Second stage of the split: out[i] = op over s of scratch[s][i].
template <typename T, class Op>
__global__ void __launch_bounds__(256)
    outer_reduce_finalize_kernel(const float* __restrict__ scratch, T* __restrict__ out,
                                 long long out_numel, int rsplit, float post_scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= out_numel) return;
  float a = scratch[i];
  for (int s = 1; s < rsplit; ++s) a = Op::combine(a, scratch[(long long)s * out_numel + i]);
  out[i] = Elem<T>::from_f(a * post_scale);
}

// Unaligned fallback (inner not a multiple of the vector width, or misaligned base):
// one thread per output column, scalar loads that are still coalesced across a warp.
template <typename T, class Op>
__global__ void __launch_bounds__(256)
    outer_reduce_scalar_kernel(const T* __restrict__ x, T* __restrict__ out, long long R,
                               long long inner, long long out_numel, float post_scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= out_numel) return;
  const long long o = i / inner, col = i % inner;
  const T* base = x + (o * R) * inner + col;
  float a = Op::identity();
  for (long long r = 0; r < R; ++r) a = Op::combine(a, Elem<T>::to_f(base[r * inner]));
  out[i] = Elem<T>::from_f(a * post_scale);
}

}  // namespace ixb
